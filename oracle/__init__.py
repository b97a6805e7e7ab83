"""CPU oracles for the GL-SDM memory operator. Test infrastructure: imported only by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs, never by gl_sdm_b200/."""
