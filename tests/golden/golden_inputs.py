"""Seeded inputs of the golden cases (shared by make_golden.py and the tests).

Shapes and seeds follow the reference's own tests for this path where one exists
(projects/gl-sdm/tests/test_chunk_memory.py:54-58,86-121; test_layer_stack.py:143-176;
test_global_memory.py:27-73; test_native_memory.py:52-106); the remaining cases are
operator-shaped variations (ties, odd sizes, hot slots). Inputs are drawn on the CPU with
torch.manual_seed so every machine with the same torch build rebuilds identical bits; the
stored float64 checksums catch a generator that ever differs.
"""
import torch
import torch.nn.functional as F

ROUTED_CASES = ("ties_zero", "colliding_tiny", "production_bank", "factor512", "signed_zero_ties",
                "c2_like", "wide_k32", "width_gt_half", "odd_half", "bf16_ties", "nan_inf_scores")
PROPOSE_CASES = ("c1_like", "two_layers", "hot_slots")


def checksum(t):
    # NaN and infinities count as fixed finite values so that the sum still pins the draw
    return float(torch.nan_to_num(t.double(), nan=7.0, posinf=11.0, neginf=-13.0).sum().item())


def routed_case(name):
    """-> (memory [B,H,S,D] fp32, scores [B,T,H,2*half] fp32, width)"""
    if name == "ties_zero":  # test_chunk_memory.py:54-58
        return torch.zeros(1, 2, 16, 3), torch.zeros(1, 5, 2, 8), 4
    if name == "colliding_tiny":  # test_chunk_memory.py:86-101
        torch.manual_seed(42)
        return torch.randn(2, 2, 16, 8), torch.randn(2, 17, 2, 8), 2
    if name == "production_bank":  # test_chunk_memory.py:104-121
        torch.manual_seed(42)
        memory = torch.randn(2, 8, 4096, 64)
        return memory, torch.randn(2, 65, 8, 128).bfloat16().float(), 8
    if name == "factor512":  # test_layer_stack.py:143-176
        torch.manual_seed(7)
        memory = torch.randn(1, 1, 262144, 64)
        scores = torch.randn(1, 3, 1, 1024)
        scores[:, 0].zero_()
        scores[:, 2].floor_()
        return memory, scores, 8
    if name == "signed_zero_ties":
        torch.manual_seed(11)
        memory = torch.randn(1, 2, 256, 4)
        scores = torch.randint(-2, 3, (1, 40, 2, 32)).float()
        scores[:, ::3] = scores[:, ::3] * -0.0  # whole rows of mixed +0.0 / -0.0
        scores[:, 1::3, :, ::2] *= -1.0
        return memory, scores, 4
    if name == "c2_like":
        torch.manual_seed(1234)
        memory = torch.randn(1, 8, 16384, 64) * 0.02
        x = torch.randn(64, 512).bfloat16()
        w = (torch.randn(8 * 256, 512) * 0.02).bfloat16()
        scores = (x.float() @ w.float().T).bfloat16().float().view(1, 64, 8, 256)
        return memory, scores, 16
    if name == "wide_k32":
        torch.manual_seed(5)
        return torch.randn(1, 1, 4096, 128), torch.randn(1, 32, 1, 128), 32
    if name == "width_gt_half":
        torch.manual_seed(6)
        return torch.randn(1, 1, 16, 8), torch.randn(1, 9, 1, 8), 6
    if name == "odd_half":
        torch.manual_seed(8)
        return torch.randn(2, 3, 36, 5), torch.randn(2, 7, 3, 12), 3
    if name == "bf16_ties":
        torch.manual_seed(9)
        memory = torch.randn(2, 2, 1024, 16)
        scores = (torch.randn(2, 33, 2, 64) * 0.25).bfloat16().float()
        scores = (scores * 4).round() / 4  # coarse grid: many exact ties at every boundary
        return memory, scores, 8
    if name == "nan_inf_scores":  # torch ranks NaN above +inf; sums with NaN are NaN and rank first
        torch.manual_seed(13)
        memory = torch.randn(1, 2, 256 * 256, 4)
        scores = torch.randn(1, 24, 2, 512)
        mask = torch.rand(scores.shape)
        scores[mask < 0.01] = float("nan")
        scores[(mask > 0.01) & (mask < 0.02)] = float("inf")
        scores[(mask > 0.02) & (mask < 0.03)] = float("-inf")
        scores[0, 0, 0, :256] = float("nan")
        scores[0, 1] = torch.randn(2, 512)          # a clean row among them
        return memory, scores, 8
    raise KeyError(name)


def propose_case(name):
    """Inputs of a write proposal + commit: scores for each proposing layer, gates, targets."""
    if name == "c1_like":
        torch.manual_seed(1234)
        B, T, H, half, D, K = 2, 32, 4, 64, 64, 8
        layers, C, L = [0], 512, 1
    elif name == "two_layers":
        torch.manual_seed(77)
        B, T, H, half, D, K = 1, 16, 2, 8, 16, 4
        layers, C, L = [1, 3], 16, 4
    elif name == "hot_slots":
        torch.manual_seed(3)
        B, T, H, half, D, K = 1, 1024, 1, 2, 32, 2
        layers, C, L = [0], 1024, 1
    else:
        raise KeyError(name)
    memory = torch.randn(B, H, half * half, D) * 0.02
    scores = torch.randn(B, T, H, 2 * half).bfloat16().float()
    extra = [torch.randn(B, T, H, 2 * half).bfloat16().float() for _ in layers[1:]]
    target = torch.randn(B, T, H, D) * 0.02
    beta = torch.randn(B, T, H).sigmoid()
    log_decay = -F.softplus(torch.randn(B, T, H) - 4)
    return dict(memory=memory, scores=scores, extra_scores=extra, target=target, beta=beta,
                log_decay=log_decay, width=K, chunk_size=C, num_layers=L, layers=layers, offset=0)


def commit_random_bank(shape):
    torch.manual_seed(42)
    return torch.randn(shape)


def commit_cases():
    """name -> (bank shape, addresses, deltas, keys or None)"""
    torch.manual_seed(21)
    cases = {
        # test_native_memory.py:95-106 / test_global_memory.py:69-73
        "cancellation": ((1, 1, 4, 1), torch.tensor([0, 3, 0, 0, 3]),
                         torch.tensor([[1e8], [0.125], [-1e8], [1.0], [0.25]]), None),
        "unrelated": ((1, 1, 4, 1), torch.tensor([0, 3]), torch.tensor([[1e8], [0.125]]), None),
        # test_chunk_memory.py:43-51
        "keyed_order": ((1, 1, 4, 1), torch.tensor([3, 3, 3]), torch.tensor([[1e8], [-1e8], [0.125]]),
                        torch.tensor([30, 31, 32])),
        "keyed_order_permuted": ((1, 1, 4, 1), torch.tensor([3, 3, 3]), torch.tensor([[0.125], [1e8], [-1e8]]),
                                 torch.tensor([32, 30, 31])),
        "random_duplicates": ((2, 1, 4, 3), torch.randint(0, 8, (20,)), torch.randn(20, 3), None),
    }
    return cases


def token_case():
    """test_native_memory.py:52-92 (inputs drawn on the CPU)."""
    torch.manual_seed(91)
    memory = torch.randn(3, 2, 67, 37)
    return dict(
        memory=memory,
        requests=torch.tensor([2, 0]),
        indices=torch.tensor([[[0, 4, 66], [1, 5, 8]], [[2, 3, 9], [0, 11, 66]]]),
        weights=torch.randn(2, 2, 3).softmax(-1),
        targets=torch.randn(2, 2, 37),
        beta=torch.full((2, 2, 1), 0.3),
        log_decay=torch.full((2, 2, 1), -0.12),
        mass=torch.tensor([0.0, 0.7]),
    )


GRAD_CASES = ("grad_tiny", "grad_c1")


def grad_case(name):
    """Inputs of the routed-read gradient cases (projects/gl-sdm/tests/test_chunk_memory.py:86-121
    check the same gradients on the reference's native path)."""
    if name == "grad_tiny":
        torch.manual_seed(42)
        return torch.randn(2, 2, 16, 8), torch.randn(2, 17, 2, 8), 2
    if name == "grad_c1":
        torch.manual_seed(4242)
        return torch.randn(2, 4, 4096, 64) * 0.02, torch.randn(2, 16, 4, 128).bfloat16().float(), 8
    raise KeyError(name)


def cotangents(name, readings_shape, weights_shape):
    g = torch.Generator().manual_seed(len(name) + 100)
    return torch.randn(readings_shape, generator=g), torch.randn(weights_shape, generator=g)


def chain_case():
    """A tiny write chain (read -> gather -> delta -> commit) with colliding addresses."""
    g = torch.Generator().manual_seed(99)
    B, T, H, half, D, K = 1, 6, 2, 4, 8, 2
    return dict(memory=torch.randn(B, H, half * half, D, generator=g), scores=torch.randn(B, T, H, 2 * half, generator=g),
                target=torch.randn(B, T, H, D, generator=g), beta=torch.rand(B, T, H, generator=g),
                log_decay=-torch.rand(B, T, H, generator=g) * 0.3, width=K,
                cotangent=torch.randn(B, H, half * half, D, generator=g))


STEP_CASES = ("c1_step", "c2_chunk_step")


def c1_step_case(name="c1_step"):
    """Bank and per-(epoch, layer) inputs of a benchmark configuration with per-request banks,
    drawn on the CPU so that every machine rebuilds the same tensors: "c1_step" is all of c1
    (2 x 1024 tokens, one layer), "c2_chunk_step" one request and one 512-token chunk of c2
    (eight global layers writing into one commit)."""
    import bench_workloads as workloads
    w = workloads.WORKLOADS["c1"] if name == "c1_step" else workloads.WORKLOADS["c2"].scaled(sequences=1, seq_len=512)
    values = workloads.make_bank(w, "cpu")
    inputs = [[workloads.make_epoch_inputs(w, "cpu", 1000 + 100 * e + layer) for layer in range(w.global_layers)]
              for e in range(w.epochs)]
    return w, values, inputs


def c1_step_digest(bank, readings):
    """What the fixture keeps of a step's results: float64 sums per (request, head) and 256
    sampled rows of the banks, the same for the readings."""
    g = torch.Generator().manual_seed(5)
    bank, readings = bank.detach().cpu(), readings.detach().cpu()
    flat = bank.flatten(0, 2)
    rows_at = torch.randint(0, flat.shape[0], (256,), generator=g)
    read_flat = readings.flatten(0, 2)
    read_at = torch.randint(0, read_flat.shape[0], (256,), generator=g)
    return dict(bank_sum=bank.double().sum((2, 3)).numpy(), bank_abs=bank.double().abs().sum((2, 3)).numpy(),
                rows_at=rows_at.numpy(), rows=flat[rows_at].numpy(),
                readings_sum=readings.double().sum((1, 3)).numpy(), read_at=read_at.numpy(),
                read_rows=read_flat[read_at].numpy())


def assert_c1_step(bank, readings, gold, rtol):
    """Compare a step's results with the stored digest of the reference's."""
    import numpy as np
    digest = c1_step_digest(bank, readings)
    assert np.array_equal(digest["rows_at"], gold["rows_at"]) and np.array_equal(digest["read_at"], gold["read_at"])
    np.testing.assert_allclose(digest["rows"], gold["rows"], rtol=rtol, atol=1e-6)
    np.testing.assert_allclose(digest["read_rows"], gold["read_rows"], rtol=rtol, atol=1e-6)
    for k in ("bank_sum", "bank_abs", "readings_sum"):
        np.testing.assert_allclose(digest[k], gold[k], rtol=1e-6, atol=1e-4, err_msg=k)
