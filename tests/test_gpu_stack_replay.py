"""Call-level replay of a reference stack forward through the CUDA path.

tests/golden/stack_trace_<dtype>.npz holds every routed_read and commit call the reference's
gl_sdm/layers/stack.py made during a prefill of its alternating local/global stack (recorded
by tests/golden/make_stack_trace.py with the reference's torch path). Each call is replayed
with exactly the recorded inputs through gl_sdm_b200.memory (the functions stack.py binds to
after gl_sdm_b200.install): routes must be bit-exact, readings within atol 1e-6 / rtol 1e-5,
committed banks bit-exact (every address receives far fewer than 256 entries)."""
import types

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_recorded_call_is_reproduced(native, dtype):
    from gl_sdm_b200.memory import MemoryView, WriteProposal, commit, merge, routing
    t = load_golden(f"stack_trace_{dtype}")
    block = types.SimpleNamespace(attn=types.SimpleNamespace(reference=False, backend="urm"))
    banks = {}

    def bank(i):
        if i not in banks:
            banks[i] = torch.from_numpy(t[f"bank{i}"]).to(DEV)
        return banks[i]

    assert int(t["reads"]) == 12 and int(t["commits"]) == 2
    ties = 0
    for i in range(int(t["reads"])):
        scores = torch.from_numpy(t[f"read{i}_scores"]).to(DEV)
        readings, index, weights = routing.routed_read(block, bank(int(t[f"read{i}_bank"])), scores, int(t[f"read{i}_width"]))
        np.testing.assert_array_equal(index.cpu().numpy(), t[f"read{i}_index"].astype(np.int64))
        np.testing.assert_allclose(weights.cpu().numpy(), t[f"read{i}_weights"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(readings.cpu().numpy(), t[f"read{i}_readings"], rtol=1e-5, atol=1e-6)
        s = np.sort(t[f"read{i}_scores"].reshape(-1, 2, scores.shape[-1] // 2), axis=-1)
        width = int(t[f"read{i}_width"])
        ties += int((s[..., -width] == s[..., -width - 1]).sum())
    if dtype == "bfloat16":
        assert ties > 0, "the bf16 trace is expected to contain exact ties at the factor boundary"
    for i in range(int(t["commits"])):
        view = MemoryView(bank(int(t[f"commit{i}_bank"])), version=i)
        proposals = [WriteProposal(i, torch.from_numpy(t[f"commit{i}_addresses{j}"]).to(DEV),
                                   torch.from_numpy(t[f"commit{i}_deltas{j}"]).to(DEV), view.lineage,
                                   torch.from_numpy(t[f"commit{i}_keys{j}"]).to(DEV))
                     for j in range(int(t[f"commit{i}_proposals"]))]
        before = view.values.clone()
        after = commit(view, merge(view, proposals), backend="urm")
        assert after.version == i + 1
        np.testing.assert_array_equal(after.values.cpu().numpy(), t[f"bank{int(t[f'commit{i}_result'])}"])
        assert torch.equal(view.values, before)
    native.raise_on_device_status(DEV)
