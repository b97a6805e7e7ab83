"""Pin the numpy oracle (oracle/sdm_oracle.py) and the torch CPU port (oracle/torch_port.py)
against outputs of the reference itself (tests/golden/*.npz, made by make_golden.py)."""
import numpy as np
import pytest
import torch

import golden_inputs as gi
from conftest import load_golden
from oracle import sdm_oracle as oracle
from oracle import torch_port as port


def _inputs_match(gold, memory, scores):
    np.testing.assert_allclose(gold["checksum"], [gi.checksum(memory), gi.checksum(scores)], rtol=1e-12)


@pytest.mark.parametrize("name", gi.ROUTED_CASES)
def test_routed_read_matches_reference(name):
    gold = load_golden(f"routed_{name}")
    memory, scores, width = gi.routed_case(name)
    _inputs_match(gold, memory, scores)
    readings, index, weights = oracle.routed_read(memory.numpy(), scores.numpy(), width)
    assert np.array_equal(index, gold["index"].astype(np.int64))
    np.testing.assert_allclose(weights, gold["weights"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(readings, gold["readings"], rtol=1e-5, atol=1e-6)
    p_read, p_index, p_weights = port.routed_read(memory, scores, width)
    assert np.array_equal(p_index.numpy(), gold["index"].astype(np.int64))
    np.testing.assert_allclose(p_weights.numpy(), gold["weights"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(p_read.numpy(), gold["readings"], rtol=1e-5, atol=1e-6)


def test_reference_tie_fixture_values():
    """projects/gl-sdm/tests/test_chunk_memory.py:54-58 as literal values."""
    _, index, weights = oracle.routed_read(np.zeros((1, 2, 16, 3), np.float32), np.zeros((1, 5, 2, 8), np.float32), 4)
    assert np.array_equal(index, np.broadcast_to(np.arange(12, 16), (1, 5, 2, 4)))
    assert np.array_equal(weights, np.full_like(weights, 0.25))


@pytest.mark.parametrize("name", gi.PROPOSE_CASES)
def test_propose_and_commit_match_reference(name):
    gold = load_golden(f"propose_{name}")
    case = gi.propose_case(name)
    memory = case["memory"].numpy()
    _inputs_match(gold, case["memory"], case["scores"])
    all_addr, all_delta, all_keys = [], [], []
    for j, layer in enumerate(case["layers"]):
        scores = case["scores"] if j == 0 else case["extra_scores"][j - 1]
        addr, delta, keys = oracle.propose(memory, scores.numpy(), case["width"], case["target"].numpy(),
                                           case["beta"].numpy(), case["log_decay"].numpy(), None, case["offset"],
                                           layer, case["chunk_size"], case["num_layers"])
        assert np.array_equal(addr, gold[f"addresses{j}"]) and np.array_equal(keys, gold[f"keys{j}"])
        np.testing.assert_allclose(delta, gold[f"deltas{j}"], rtol=1e-5, atol=1e-8)
        all_addr.append(addr), all_delta.append(delta), all_keys.append(keys)
        p = port.propose(case["memory"], scores, case["width"], case["target"], case["beta"], case["log_decay"],
                         None, case["offset"], layer, case["chunk_size"], case["num_layers"])
        assert np.array_equal(p[0].numpy(), gold[f"addresses{j}"]) and np.array_equal(p[2].numpy(), gold[f"keys{j}"])
        np.testing.assert_allclose(p[1].numpy(), gold[f"deltas{j}"], rtol=1e-5, atol=1e-8)
    # commit the reference's own deltas so this check is independent of the exp rounding above
    deltas = np.concatenate([gold[f"deltas{j}"] for j in range(len(case["layers"]))])
    after = oracle.commit(memory, np.concatenate(all_addr), deltas, np.concatenate(all_keys))
    flat = after.reshape(-1, memory.shape[-1])
    np.testing.assert_array_equal(flat[gold["touched"]], gold["touched_rows"])
    untouched = np.ones(flat.shape[0], bool)
    untouched[gold["touched"]] = False
    np.testing.assert_array_equal(flat[untouched], memory.reshape(flat.shape)[untouched])
    ported = port.commit(case["memory"], torch.from_numpy(np.concatenate(all_addr)), torch.from_numpy(deltas),
                         torch.from_numpy(np.concatenate(all_keys)))
    np.testing.assert_array_equal(ported.flatten(0, 2).numpy()[gold["touched"]], gold["touched_rows"])


def test_commit_known_answers():
    gold = load_golden("commit_cases")
    for name, (shape, idx, delta, keys) in gi.commit_cases().items():
        bank = gi.commit_random_bank(shape).numpy() if name == "random_duplicates" else np.zeros(shape, np.float32)
        out = oracle.commit(bank, idx.numpy(), delta.numpy(), None if keys is None else keys.numpy())
        np.testing.assert_array_equal(out, gold[f"{name}_out"])
        np.testing.assert_allclose(out, gold[f"{name}_dense"], rtol=1e-6, atol=1e-6) if name == "random_duplicates" else None
        ported = port.commit(torch.from_numpy(bank), idx, delta, keys)
        np.testing.assert_array_equal(ported.numpy(), gold[f"{name}_out"])
    # literal values of projects/gl-sdm/tests/test_native_memory.py:95-106 and test_chunk_memory.py:43-51
    assert gold["cancellation_out"].reshape(-1).tolist() == [1.0, 0.0, 0.0, 0.375]
    assert gold["keyed_order_out"].reshape(-1)[3] == 0.125
    np.testing.assert_array_equal(gold["keyed_order_out"], gold["keyed_order_permuted_out"])
    dense = oracle.commit_dense(gi.commit_random_bank((2, 1, 4, 3)).numpy(), gi.commit_cases()["random_duplicates"][1].numpy(),
                                gi.commit_cases()["random_duplicates"][2].numpy())
    np.testing.assert_allclose(dense, gold["random_duplicates_dense"], rtol=1e-6, atol=1e-6)


def test_token_api_matches_reference():
    gold = load_golden("token_api")
    t = {k: v.numpy() for k, v in gi.token_case().items()}
    read = oracle.token_read(t["memory"], t["requests"], t["indices"], t["weights"])
    np.testing.assert_allclose(read, gold["read"], rtol=1e-6, atol=1e-7)
    addr, delta = oracle.token_propose(t["memory"], t["requests"], t["indices"], t["weights"], t["targets"],
                                       t["beta"], t["log_decay"], t["mass"])
    assert np.array_equal(addr, gold["addresses"])
    np.testing.assert_allclose(delta, gold["deltas"], rtol=1e-5, atol=1e-7)
    _, delta2 = oracle.token_propose(t["memory"], t["requests"], t["indices"], t["weights"], t["targets"] * 2,
                                     t["beta"], t["log_decay"], 1 - t["mass"])
    updated = oracle.commit(t["memory"], np.concatenate([addr, addr]), np.concatenate([gold["deltas"], gold["deltas2"]]))
    np.testing.assert_array_equal(updated, gold["updated"])
    np.testing.assert_allclose(delta2, gold["deltas2"], rtol=1e-5, atol=1e-7)


def test_flat_selection_rule_equals_product_key_rule():
    """The product-key selection equals a flat top-k of s[a] = left[a // half] + right[a % half]
    under (score descending, slot descending) - the form the streaming kernels implement."""
    rng = np.random.default_rng(0)
    for half, width in ((4, 2), (8, 4), (16, 8), (6, 3)):
        scores = rng.integers(-2, 3, size=(1, 50, 2, 2 * half)).astype(np.float32)
        scores[:, ::5] *= np.float32(-0.0)
        index, weights = oracle.select_routes(scores, width)
        left, right = scores[..., :half], scores[..., half:]
        flat = (left[..., :, None] + right[..., None, :]).reshape(-1, half * half)
        slot, score = oracle.top_routes(flat, width)
        slot, w = oracle.canonical_routes(slot, score)
        assert np.array_equal(slot.reshape(index.shape), index)
        np.testing.assert_allclose(w.reshape(weights.shape), weights, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_oracle_replays_the_recorded_stack_calls(dtype):
    """Every routed_read / commit call of a reference stack prefill (tests/golden/stack_trace_*)."""
    t = load_golden(f"stack_trace_{dtype}")
    for i in range(int(t["reads"])):
        readings, index, weights = oracle.routed_read(t[f"bank{int(t[f'read{i}_bank'])}"], t[f"read{i}_scores"],
                                                      int(t[f"read{i}_width"]))
        assert np.array_equal(index, t[f"read{i}_index"])
        np.testing.assert_allclose(weights, t[f"read{i}_weights"], rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(readings, t[f"read{i}_readings"], rtol=1e-5, atol=1e-6)
    for i in range(int(t["commits"])):
        n = int(t[f"commit{i}_proposals"])
        cat = lambda name: np.concatenate([t[f"commit{i}_{name}{j}"] for j in range(n)])  # noqa: E731
        out = oracle.commit(t[f"bank{int(t[f'commit{i}_bank'])}"], cat("addresses"), cat("deltas"), cat("keys"))
        np.testing.assert_array_equal(out, t[f"bank{int(t[f'commit{i}_result'])}"])


@pytest.mark.parametrize("name", gi.GRAD_CASES)
def test_oracle_backward_matches_reference_autograd(name):
    gold = load_golden("gradients")
    memory, scores, width = gi.grad_case(name)
    readings, index, weights = oracle.routed_read(memory.numpy(), scores.numpy(), width)
    cot_r, cot_w = gi.cotangents(name, readings.shape, weights.shape)
    grad_routes, grad_memory = oracle.routed_read_backward(memory.numpy(), index, weights, cot_r.numpy(), cot_w.numpy())
    grad_scores = oracle.scatter_route_gradients(grad_routes, index, scores.shape[-1] // 2)
    np.testing.assert_allclose(grad_scores, gold[f"{name}_grad_scores"], rtol=1e-4, atol=1e-6)
    flat = grad_memory.reshape(-1, memory.shape[-1])
    np.testing.assert_allclose(flat[gold[f"{name}_touched"]], gold[f"{name}_grad_rows"], rtol=1e-4, atol=1e-6)
    untouched = np.ones(flat.shape[0], bool)
    untouched[gold[f"{name}_touched"]] = False
    assert not flat[untouched].any()


@pytest.mark.parametrize("name", gi.STEP_CASES)
def test_cpu_port_runs_the_c1_step_like_the_reference(name):
    """The timed CPU baseline of the per-request configurations (bench.PortMemory behind
    bench.api_step) against the same step driven through the reference's gl_sdm.memory."""
    import bench
    gold = load_golden(name)
    w, values, inputs = gi.c1_step_case(name)
    drawn = [gi.checksum(values)] + [gi.checksum(x[k]) for layers in inputs for x in layers for k in sorted(x)]
    np.testing.assert_allclose(drawn, gold["checksum"], rtol=1e-12)
    readings, view = bench.api_step(w, values.clone(), inputs, bench.PortMemory())
    assert view.version == w.epochs
    gi.assert_c1_step(view.values, readings, gold, rtol=1e-5)
