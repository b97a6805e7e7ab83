"""A minimal in-process stand-in for torch.distributed: R virtual ranks run as Python threads
and meet at barriers. It lets one GPU (or the CPU) execute the R-rank exchange of
ShardedBankOperator with the real kernels; all launches share the default stream, so no
kernel ever waits on another one. Test infrastructure only."""
import threading

import torch


class ThreadWorld:
    def __init__(self, world):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.slots = [None] * world
        self.local = threading.local()

    def rank_view(self, rank):
        return _RankDist(self, rank)

    def run(self, fn):
        """fn(rank, dist) on every virtual rank; returns the list of results (re-raises errors)."""
        results, errors = [None] * self.world, []

        def body(rank):
            try:
                results[rank] = fn(rank, self.rank_view(rank))
            except BaseException as exc:  # noqa: BLE001
                errors.append(exc)
                self.barrier.abort()

        threads = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return results


class _RankDist:
    def __init__(self, world, rank):
        self.w, self.rank = world, rank

    def get_world_size(self, group=None):
        return self.w.world

    def get_rank(self, group=None):
        return self.rank

    def _exchange(self, tensor):
        self.w.slots[self.rank] = tensor
        self.w.barrier.wait()
        pieces = list(self.w.slots)
        self.w.barrier.wait()
        return pieces

    def all_gather_into_tensor(self, out, inp, group=None):
        pieces = self._exchange(inp)
        out.view(self.w.world, -1).copy_(torch.stack([p.reshape(-1) for p in pieces]))
        self.w.barrier.wait()

    def reduce_scatter_tensor(self, out, inp, group=None):
        pieces = self._exchange(inp)
        n = out.numel()
        total = torch.zeros_like(out).view(-1)
        for p in pieces:
            total += p.reshape(-1)[self.rank * n:(self.rank + 1) * n]
        out.copy_(total.view_as(out))
        self.w.barrier.wait()

    def all_gather(self, outs, inp, group=None):
        pieces = self._exchange(inp)
        for o, p in zip(outs, pieces):
            o.copy_(p)
        self.w.barrier.wait()

    def all_to_all_single(self, out, inp, group=None):
        pieces = self._exchange(inp)
        n = out.numel() // self.w.world
        out.view(self.w.world, n).copy_(torch.stack([p.reshape(self.w.world, n)[self.rank] for p in pieces]))
        self.w.barrier.wait()

    def peer_memory(self, numel, device, group=None):
        """float32 [numel] of this rank and the addresses of every rank's: the virtual ranks share
        one process and one GPU, so plain allocations are each other's "peer memory"."""
        mine = torch.empty(numel, dtype=torch.float32, device=device)
        pieces = self._exchange(mine)
        self.w.barrier.wait()
        self.w.local.__dict__.setdefault("kept", []).append(pieces)      # the peers' tensors must outlive their users
        return mine, [p.data_ptr() for p in pieces]
