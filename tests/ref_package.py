"""Load the staged reference package (oracle/_ref, see oracle/make_ref.py) under several bindings.

Test infrastructure. The reference resolves ``gl_sdm.memory`` and its backends through
``sys.modules`` - partly at import time (layers/stack.py:8, layers/global_layer.py:5-6),
partly inside functions (model.py:33-34,58; memory/routing.py:47; memory/transactions.py:82)
- so one process can hold the same unmodified source bound several ways:

  "reference"  the reference's own memory package (its torch path is the oracle);
  "shim"       gl_sdm_b200.install: the whole memory package replaced (package seam);
  "fused"      the same, plus GlobalLayer.propose replaced by the fused write proposal;
  "seam"       the reference's own memory package with only its two native backend modules,
               backends.urm and backends.commit, replaced (backend seam, config "urm").

Each binding owns its module objects; ``with binding:`` makes them the ones ``sys.modules``
serves, which the function-level imports need while that binding's model runs.
"""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def available():
    return os.path.exists(os.path.join(REF, "gl_sdm", "__init__.py"))


def require():
    if not available():
        pytest.skip("the reference package is not staged under oracle/_ref (python oracle/make_ref.py <checkout>)")


def _ours(name):
    return name == "gl_sdm" or name.startswith("gl_sdm.")


class Binding:
    def __init__(self, kind):
        self.kind, self.modules, self._saved = kind, {}, []

    def __enter__(self):
        self._saved.append({n: m for n, m in sys.modules.items() if _ours(n)})
        for n in list(self._saved[-1]):
            del sys.modules[n]
        sys.modules.update(self.modules)
        return self

    def __exit__(self, *exc):
        self.modules = {n: m for n, m in sys.modules.items() if _ours(n)}   # keep late imports
        for n in list(self.modules):
            del sys.modules[n]
        sys.modules.update(self._saved.pop())
        return False

    def module(self, name):
        with self:
            return importlib.import_module(name)

    def create_model(self, cfg):
        with self:
            return importlib.import_module("gl_sdm.model").create_model(cfg)


def load(kind):
    require()
    if REF not in sys.path:
        sys.path.insert(0, REF)
    binding = Binding(kind)
    with binding:
        if kind in ("shim", "fused"):
            from gl_sdm_b200 import install
            install.install()
        elif kind == "seam":
            from gl_sdm_b200.memory.backends import commit, urm
            sys.modules["gl_sdm.memory.backends.urm"] = urm
            sys.modules["gl_sdm.memory.backends.commit"] = commit
        elif kind != "reference":
            raise ValueError(kind)
        importlib.import_module("gl_sdm.model")
        importlib.import_module("gl_sdm.layers.stack")
        if kind == "fused":
            from gl_sdm_b200.layers import install_fused_proposals
            install_fused_proposals(importlib.import_module("gl_sdm.layers.global_layer"))
        memory = importlib.import_module("gl_sdm.memory")
        origin = os.path.dirname(os.path.abspath(memory.__file__))
        if kind in ("shim", "fused"):
            assert origin.startswith(os.path.join(ROOT, "gl_sdm_b200")), origin
        else:
            assert origin.startswith(REF), origin
    return binding


def stack_config(**overrides):
    """The reference model at the widths of benchmark configuration 2 (hidden 512, 8 heads of
    64, 16 alternating local/global layers, 16,384 slots, 16 reads and writes, 512-token
    chunks, window 256); tests shrink what they do not need."""
    cfg = dict(arch_type="gl_sdm", vocab_size=32000, hidden_size=512, head_dim=64, num_hidden_layers=16,
               intermediate_size=2048, dtype="float32", gl_layer_pattern=["local", "global"], gl_local_window=256,
               gl_chunk_size=512, gl_slots=16384, gl_reads=16, gl_writes=16, gl_memory_backend="torch")
    cfg.update(overrides)
    return cfg
