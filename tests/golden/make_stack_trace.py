"""Record every memory-operator call of a reference GL-SDM stack forward (CPU, torch path).

    python tests/golden/make_stack_trace.py /path/to/GL-SDM

Runs the reference's own 16-layer-style stack (gl_sdm/layers/stack.py, alternating local /
global layers) at a small width through model.prefill, with routing.routed_read and
transactions.commit wrapped, and stores each call's inputs and outputs in
stack_trace_<dtype>.npz. tests/test_gpu_stack_replay.py replays the calls one by one through
the CUDA path ("teacher forcing": every call sees exactly the reference's inputs, so one
rounding difference cannot change a later route). The bf16 variant matters because its
factor scores are bf16 GEMM outputs: exact ties at the selection boundaries are frequent.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIG = dict(arch_type="gl_sdm", vocab_size=64, hidden_size=64, head_dim=16, num_hidden_layers=4,
              gl_layer_pattern=["local", "global"], gl_slots=256, gl_reads=4, gl_writes=4, gl_chunk_size=8,
              gl_local_window=6, gl_memory_backend="torch", intermediate_size=128, seq_len=20)


def main(root):
    sys.path.insert(0, os.path.join(root, "projects", "gl-sdm", "src"))
    from gl_sdm.model import create_model
    import gl_sdm.memory.routing as routing
    import gl_sdm.layers.stack as stack
    for dtype in ("float32", "bfloat16"):
        torch.manual_seed(1234)
        model = create_model({**CONFIG, "dtype": dtype}).eval()
        ids = torch.randint(64, (2, 20))
        rec, banks = {}, {}
        counters = {"read": 0, "commit": 0}

        def bank_id(values, fresh=False):
            # storage addresses are recycled once an old version is freed: a commit's result
            # is always registered as a new bank, lookups use the latest bank at an address
            key = values.data_ptr()
            if fresh or key not in banks:
                banks[key] = sum(1 for name in rec if name.startswith("bank"))
                rec[f"bank{banks[key]}"] = values.detach().numpy().copy()
            return banks[key]

        original_read = routing.routed_read
        original_commit = stack.commit

        def read(block, memory, scores, width, physical=None):
            out = original_read(block, memory, scores, width, physical)
            i = counters["read"]
            counters["read"] += 1
            rec[f"read{i}_bank"] = np.array(bank_id(memory))
            rec[f"read{i}_scores"] = scores.detach().numpy().copy()
            rec[f"read{i}_width"] = np.array(width)
            rec[f"read{i}_readings"] = out[0].detach().numpy().copy()
            rec[f"read{i}_index"] = out[1].numpy().astype(np.int32)
            rec[f"read{i}_weights"] = out[2].detach().numpy().copy()
            return out

        def commit(view, buffer, **kw):
            result = original_commit(view, buffer, **kw)
            i = counters["commit"]
            counters["commit"] += 1
            rec[f"commit{i}_bank"] = np.array(bank_id(view.values))
            rec[f"commit{i}_proposals"] = np.array(len(buffer.proposals))
            for j, p in enumerate(buffer.proposals):
                rec[f"commit{i}_addresses{j}"] = p.addresses.numpy().copy()
                rec[f"commit{i}_deltas{j}"] = p.deltas.detach().float().numpy().copy()
                rec[f"commit{i}_keys{j}"] = p.sort_keys.numpy().copy()
            rec[f"commit{i}_result"] = np.array(bank_id(result.values, fresh=True))
            return result

        routing.routed_read, stack.commit = read, commit
        try:
            with torch.inference_mode():
                logits, cache = model.prefill(ids)
        finally:
            routing.routed_read, stack.commit = original_read, original_commit
        rec["reads"], rec["commits"] = np.array(counters["read"]), np.array(counters["commit"])
        np.savez_compressed(os.path.join(HERE, f"stack_trace_{dtype}.npz"), **rec)
        print(dtype, counters, "banks", sum(1 for name in rec if name.startswith("bank")), "final version",
              cache[0].view.version)


if __name__ == "__main__":
    main(sys.argv[1])
