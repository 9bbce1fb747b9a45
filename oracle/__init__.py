"""TEST INFRASTRUCTURE: CPU restatement of the reference's kernels (oracle.c) and, when it was built from a DAPHNE
source tree, the reference's own CPU kernels (oracle/_ref).  Only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline may import this package; nothing under daphne_b200/ does."""
