"""Where an explicitly requested oracle (``reference=True``) is looked up.

The shipped package contains one implementation, the CUDA one. The reference API has a
``reference`` switch (gl_sdm/memory/transactions.py:69,85-88; routing.py:46) that its own
tests use to ask for an independent equation. Here that switch resolves to functions a test
harness registers; with none registered the call raises.
"""
_registered = {}


def register(**functions):
    """register(routed_read=f, commit=g, gather_rows=h, read=r, propose_write=p)"""
    _registered.update(functions)


def clear():
    _registered.clear()


def get(name):
    fn = _registered.get(name)
    if fn is None:
        raise RuntimeError(
            f"reference=True requested the '{name}' oracle, but none is registered: this package ships only "
            "the CUDA implementation (tests register an oracle through gl_sdm_b200.memory.oracle_hook)")
    return fn
