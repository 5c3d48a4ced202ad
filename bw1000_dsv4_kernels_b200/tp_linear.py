"""Column-sharded tensor-parallel W8A8 linear layer.

The [N, K] int8 weight is split on N over the G ranks of one node; the activation X [M, K] is
replicated and every rank quantises it itself (per_token_quant_int8), computes its own slab
C[:, r*N/G:(r+1)*N/G] with the int8 GEMM, and the slabs are exchanged so that every rank ends
with the full bf16 [M, N].

The reference has no collective code at all (its server ran `--tp 8` outside the repository,
README.md:104); the exchange here is NCCL over NVLink:

  * each rank's GEMM writes its slab into a slab-major buffer out_slabs[r] ([G, M, N/G], the
    layout ncclAllGather produces), `all_gather_into_tensor` fills the other slabs in place;
  * `row_major()` gives the [M, N] view consumers expect (one strided copy), or the slab-major
    buffer can be consumed directly by a following row-sharded layer.
"""
import torch


def _ext():
    import bw1000_dsv4_kernels_b200 as pkg
    return pkg.dsv4_native_ext


def column_range(rank: int, world: int, n: int):
    assert n % world == 0, "N must divide evenly over the ranks"
    per = n // world
    return rank * per, (rank + 1) * per


def peer_order(rank: int, world: int):
    """The other ranks in the order rank+1, rank+2, ... (mod world)."""
    return [(rank + 1 + d) % world for d in range(world - 1)]


class ColumnParallelW8A8Linear:
    def __init__(self, w_local, w_scale_local, rank: int = 0, world: int = 1, process_group=None):
        """w_local int8 [N/G, K], w_scale_local fp32 [N/G] (this rank's rows of the weight)."""
        self.w, self.w_scale = w_local, w_scale_local
        self.rank, self.world, self.pg = rank, world, process_group
        self.n_local = w_local.shape[0]
        self._buf = None

    def _slabs(self, m, device):
        shape = (self.world, m, self.n_local)
        if self._buf is None or self._buf.shape != shape or self._buf.device != device:
            self._buf = torch.empty(shape, dtype=torch.bfloat16, device=device)
        return self._buf

    def local_gemm(self, x, out=None):
        """quantise + GEMM for this rank's columns -> bf16 [M, N/G] (written into `out` if given)."""
        ext = _ext()
        q, s = ext.per_token_quant_int8(x)
        if out is None:
            return ext.w8a8_scaled_gemm(q, self.w, s, self.w_scale)
        ext.w8a8_gemm_into(q, self.w, s, self.w_scale, out, 0)
        return out

    def forward_slabs(self, x):
        """-> bf16 [G, M, N/G]: slab r holds columns [r*N/G, (r+1)*N/G) of the result."""
        slabs = self._slabs(x.shape[0], x.device)
        self.local_gemm(x, out=slabs[self.rank])
        if self.world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(slabs.view(-1), slabs[self.rank].reshape(-1), group=self.pg)
        return slabs

    def forward(self, x):
        """-> bf16 [M, N] row-major."""
        slabs = self.forward_slabs(x)
        if self.world == 1:
            return slabs[0]
        return slabs.permute(1, 0, 2).reshape(x.shape[0], self.world * self.n_local)


class FusedColumnParallelW8A8Linear(ColumnParallelW8A8Linear):
    """Same layer with the exchange fused into the GEMM: the output [M, N] lives in symmetric
    memory (every rank's buffer is mapped into every other rank), and the GEMM's tile epilogue
    stages each bf16 tile of this rank's column slab in shared memory, 64 columns at a time, and
    sends it with TMA tile stores into all G buffers over NVLink (`w8a8_gemm_allgather`), so the
    transfer overlaps the tensor-core work tile by tile and the result is row-major without a
    gather or a permute.

    Ordering between ranks: a symmetric-memory barrier on the stream after the kernel makes every
    slab visible before anyone reads a full row.  Nothing may overwrite rows that a slower peer is
    still reading from an earlier call; with `buffers=2` (default) consecutive calls alternate
    between two output buffers, and the barrier that ends call i already proves that every rank
    has finished the work it queued before call i, i.e. its reads of call i-1's buffer, so call
    i+1 can write that buffer without a barrier in front.  The result of a call therefore stays
    valid until the call after the next one starts.  With `buffers=1` a second barrier before the
    kernel gives the same protection for a single buffer.

    Every rank sends its tiles to the peers in the order rank+1, rank+2, ... (mod G), so that at
    any moment the G senders aim at G different receivers."""

    def __init__(self, w_local, w_scale_local, rank, world, m_max, device, process_group=None, buffers: int = 2,
                 rotate_peers: bool = True):
        super().__init__(w_local, w_scale_local, rank, world, process_group)
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        assert buffers in (1, 2)
        self.n = self.n_local * world
        self._symm = symm_mem
        group = process_group if process_group is not None else dist.group.WORLD
        self.outs, self.handles, self.peer_ptrs = [], [], []
        order = peer_order(rank, world) if rotate_peers else [r for r in range(world) if r != rank]
        for _ in range(buffers):
            out = symm_mem.empty((m_max, self.n), dtype=torch.bfloat16, device=device)
            handle = symm_mem.rendezvous(out, group=group)
            ptrs = list(handle.buffer_ptrs)
            self.outs.append(out)
            self.handles.append(handle)
            self.peer_ptrs.append([int(ptrs[r]) for r in order])
        self._turn = 0

    @property
    def out(self):
        """The buffer the most recent call wrote."""
        return self.outs[(self._turn - 1) % len(self.outs)]

    def forward(self, x):
        ext = _ext()
        m = x.shape[0]
        b = self._turn % len(self.outs)
        out, handle = self.outs[b], self.handles[b]
        assert m <= out.shape[0], "batch larger than the symmetric output buffer"
        q, s = ext.per_token_quant_int8(x)
        if len(self.outs) == 1:
            handle.barrier(channel=0)
        ext.w8a8_gemm_allgather(q, self.w, s, self.w_scale, out[:m], self.rank * self.n_local, self.peer_ptrs[b])
        handle.barrier(channel=1)
        self._turn += 1
        return out[:m]
