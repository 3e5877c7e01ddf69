"""CPU oracle of the paged-attention path.  TEST INFRASTRUCTURE ONLY: imported by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs as the checker — never by the
nano_vllm_b200 package."""
