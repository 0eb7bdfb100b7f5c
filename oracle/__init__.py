"""TEST INFRASTRUCTURE, not product code.

CPU restatements of the reference's formulation of the hot-path ops, used only
as the checker by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline
and reference legs.  Nothing under nemotron_infer_b200/ imports this package.
"""
