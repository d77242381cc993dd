"""TEST INFRASTRUCTURE: CPU restatements of the decode hot path, used only as the checker (tests/,
__graft_entry__.smoke(), bench.py's CPU-baseline legs). Nothing under nanochat_b200/ imports this package."""
