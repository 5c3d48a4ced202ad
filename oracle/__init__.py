"""CPU oracle for the W8A8 linear path (test infrastructure, never shipped code).

`oracle.cpu` wraps the C restatement; `oracle.formulas` holds independent numpy/torch
formulas that the C restatement is itself checked against.
"""
