"""CPU restatement of the reference's arithmetic and the recipe that builds the reference's own emitted kernel.

Test infrastructure: imported only by tests/, by __graft_entry__.smoke() and by the baseline legs of bench.py. Nothing
in deuteron_b200/ imports it; the product has no CPU path.
"""
