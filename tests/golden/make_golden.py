"""Generate the golden vectors in this directory from the reference itself.

Run where the reference checkout is present (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/GL-SDM [routed case names ...]

It imports the reference's own gl_sdm.memory (CPU, torch path), replays the inputs of the
reference's tests for this path (tests/test_chunk_memory.py, test_layer_stack.py,
test_global_memory.py, test_native_memory.py) plus seeded operator-shaped cases, and stores
inputs and reference outputs as .npz files. Large inputs are stored as a recipe (seed and
draw order) plus a float64 checksum; golden_inputs.py rebuilds them.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import golden_inputs as gi  # noqa: E402


def main(reference_root, only=None):
    sys.path.insert(0, os.path.join(reference_root, "projects", "gl-sdm", "src"))
    from gl_sdm.memory import MemoryView, WriteProposal, commit, merge, read, propose_write
    from gl_sdm.memory.routing import torch_routed_read, gather_rows, absolute_addresses
    from gl_sdm.runtime.dense import proposal_delta

    torch.set_num_threads(8)
    out = {}

    # -- routed reads -------------------------------------------------------------------
    for name in gi.ROUTED_CASES:
        if only and name not in only:
            continue
        memory, scores, width = gi.routed_case(name)
        readings, index, weights = torch_routed_read(memory, scores, width)
        rec = {"readings": readings.numpy(), "index": index.numpy().astype(np.int32), "weights": weights.numpy(),
               "checksum": np.array([gi.checksum(memory), gi.checksum(scores)])}
        if memory.numel() + scores.numel() <= 1 << 16:
            rec["memory"], rec["scores"] = memory.numpy(), scores.numpy()
        np.savez_compressed(os.path.join(HERE, f"routed_{name}.npz"), **rec)
        out[f"routed_{name}"] = tuple(index.shape)
    for name in gi.STEP_CASES:
        if only and name in only:
            write_c1_step(reference_root, name)
            out[name] = ()
    if only and "token_gradients" in only:
        write_token_gradients(MemoryView, read, propose_write)
        out["token_gradients"] = ()
    if only:
        print("wrote", sorted(out))
        return

    # -- write proposal (global_layer.py:41-54 from the scores on) + commit ---------------
    for name in gi.PROPOSE_CASES:
        case = gi.propose_case(name)
        memory, scores = case["memory"], case["scores"]
        B, T, H, _ = scores.shape
        width, C, L = case["width"], case["chunk_size"], case["num_layers"]
        proposals, records = [], {}
        view = MemoryView(memory)
        for j, layer in enumerate(case["layers"]):
            s = scores if j == 0 else case["extra_scores"][j - 1]
            prediction, index, weights = torch_routed_read(memory, s, width)
            rows = gather_rows(memory, index)
            addresses = absolute_addresses(memory, index)
            delta = proposal_delta(rows, weights, prediction, case["target"], case["beta"].unsqueeze(-1),
                                   case["log_decay"].unsqueeze(-1), torch.ones(B, T))
            positions = torch.arange(case["offset"], case["offset"] + T).view(1, T, 1, 1)
            keys = addresses * (C * L) + positions * L + layer
            proposals.append(WriteProposal(0, addresses.flatten(), delta.flatten(0, 3), view.lineage, keys.flatten()))
            records[f"addresses{j}"] = addresses.flatten().numpy()
            records[f"keys{j}"] = keys.flatten().numpy()
            records[f"deltas{j}"] = delta.flatten(0, 3).numpy()
        after = commit(view, merge(view, proposals))
        # store the committed bank sparsely: rows that changed
        flat_before = memory.flatten(0, 2)
        flat_after = after.values.flatten(0, 2)
        touched = torch.unique(torch.cat([p.addresses for p in proposals]))
        assert torch.equal(flat_before[~torch.isin(torch.arange(flat_before.shape[0]), touched)],
                           flat_after[~torch.isin(torch.arange(flat_before.shape[0]), touched)])
        records["touched"] = touched.numpy()
        records["touched_rows"] = flat_after[touched].numpy()
        records["checksum"] = np.array([gi.checksum(memory), gi.checksum(scores)])
        np.savez_compressed(os.path.join(HERE, f"propose_{name}.npz"), **records)
        out[f"propose_{name}"] = int(touched.numel())

    # -- commit known-answer cases ----------------------------------------------------------
    rec = {}
    for name, (shape, idx, delta, keys) in gi.commit_cases().items():
        view = MemoryView(torch.zeros(shape) if name != "random_duplicates" else gi.commit_random_bank(shape))
        p = WriteProposal(0, idx, delta, view.lineage, keys)
        result = commit(view, merge(view, [p]))
        dense = commit(view, merge(view, [p]), reference=True)
        rec[f"{name}_out"] = result.values.numpy()
        rec[f"{name}_dense"] = dense.values.numpy()
    np.savez_compressed(os.path.join(HERE, "commit_cases.npz"), **rec)

    # -- gradients (reference autograd on the torch path) ----------------------------------------
    rec = {}
    for name in gi.GRAD_CASES:
        memory, scores, width = gi.grad_case(name)
        memory.requires_grad_(), scores.requires_grad_()
        readings, index, weights = torch_routed_read(memory, scores, width)
        cot_r, cot_w = gi.cotangents(name, readings.shape, weights.shape)
        g_memory, g_scores = torch.autograd.grad((readings * cot_r).sum() + (weights * cot_w).sum(), (memory, scores))
        touched = torch.unique(absolute_addresses(memory, index))
        assert g_memory.flatten(0, 2).abs().sum(-1).nonzero().numel() <= touched.numel()
        rec[f"{name}_grad_scores"] = g_scores.numpy()
        rec[f"{name}_touched"] = touched.numpy()
        rec[f"{name}_grad_rows"] = g_memory.flatten(0, 2)[touched].numpy()
    # the whole write chain: routed read -> gather -> delta -> commit, gradient of the new bank
    chain = gi.chain_case()
    memory, scores, target = (chain[k].clone().requires_grad_() for k in ("memory", "scores", "target"))
    B, T, H, _ = scores.shape
    prediction, index, weights = torch_routed_read(memory, scores, chain["width"])
    rows = gather_rows(memory, index)
    addresses = absolute_addresses(memory, index)
    delta = proposal_delta(rows, weights, prediction, target, chain["beta"].unsqueeze(-1),
                           chain["log_decay"].unsqueeze(-1), torch.ones(B, T))
    positions = torch.arange(T).view(1, T, 1, 1)
    keys = addresses * (T * 2) + positions * 2 + 1
    view = MemoryView(memory)
    after = commit(view, merge(view, [WriteProposal(0, addresses.flatten(), delta.flatten(0, 3), view.lineage, keys.flatten())]))
    grads = torch.autograd.grad((after.values * chain["cotangent"]).sum(), (memory, scores, target))
    rec["chain_after"] = after.values.detach().numpy()
    for k, g in zip(("memory", "scores", "target"), grads):
        rec[f"chain_grad_{k}"] = g.numpy()
    np.savez_compressed(os.path.join(HERE, "gradients.npz"), **rec)

    # -- token-clock API ------------------------------------------------------------------------
    t = gi.token_case()
    view = MemoryView(t["memory"])
    retrieved = read(view, t["requests"], t["indices"], t["weights"])
    p = propose_write(view, t["requests"], t["indices"], t["weights"], t["targets"], t["beta"], t["log_decay"], t["mass"])
    p2 = propose_write(view, t["requests"], t["indices"], t["weights"], t["targets"] * 2, t["beta"], t["log_decay"], 1 - t["mass"])
    updated = commit(view, merge(view, [p, p2]))
    np.savez_compressed(os.path.join(HERE, "token_api.npz"), read=retrieved.numpy(), addresses=p.addresses.numpy(),
                        deltas=p.deltas.numpy(), deltas2=p2.deltas.numpy(), updated=updated.values.numpy())
    write_token_gradients(MemoryView, read, propose_write)
    for name in gi.STEP_CASES:
        write_c1_step(reference_root, name)
    print("wrote", sorted(out), "commit_cases token_api token_gradients", *gi.STEP_CASES)


def write_c1_step(reference_root, name):
    """One whole step of a per-request-bank benchmark configuration (golden_inputs.STEP_CASES)
    driven through the reference's own gl_sdm.memory with the call sequence the
    benchmark times (bench.api_step). Stored: float64 sums per (request, head) and sampled
    rows of the final banks and of the last chunk's readings."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    import types
    import bench
    import gl_sdm.memory as reference_memory
    from gl_sdm.memory import routing as reference_routing
    w, values, inputs = gi.c1_step_case(name)
    memory = types.SimpleNamespace(MemoryView=reference_memory.MemoryView, WriteProposal=reference_memory.WriteProposal,
                                   merge=reference_memory.merge, commit=reference_memory.commit, routing=reference_routing)
    readings, view = bench.api_step(w, values.clone(), inputs, memory)
    assert view.version == w.epochs
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **gi.c1_step_digest(view.values, readings),
                        checksum=np.array([gi.checksum(values)] + [gi.checksum(x[k]) for layers in inputs for x in layers
                                                                   for k in sorted(x)]))


def write_token_gradients(MemoryView, read, propose_write):
    """Reference autograd through the token-clock read and write proposal (torch path; the
    native path's hand-written backward is gl_sdm/memory/backends/token.py:134-168)."""
    t = gi.token_case()
    names = ("memory", "weights", "targets", "beta", "log_decay", "mass")
    leaves = {k: t[k].clone().requires_grad_() for k in names}
    view = MemoryView(leaves["memory"])
    retrieved = read(view, t["requests"], t["indices"], leaves["weights"])
    p = propose_write(view, t["requests"], t["indices"], leaves["weights"], leaves["targets"], leaves["beta"],
                      leaves["log_decay"], leaves["mass"])
    cot_read, cot_delta = gi.cotangents("token", retrieved.shape, p.deltas.shape)
    rec = {}
    grads = torch.autograd.grad((retrieved * cot_read).sum(), (leaves["memory"], leaves["weights"]), retain_graph=True)
    rec["read_grad_memory"], rec["read_grad_weights"] = (g.numpy() for g in grads)
    grads = torch.autograd.grad((p.deltas * cot_delta).sum(), [leaves[k] for k in names])
    for k, g in zip(names, grads):
        rec[f"propose_grad_{k}"] = g.numpy()
    np.savez_compressed(os.path.join(HERE, "token_gradients.npz"), **rec)


if __name__ == "__main__":
    # python make_golden.py [reference root] [routed case names to (re)write; default: everything]
    main(sys.argv[1], set(sys.argv[2:]) or None)
