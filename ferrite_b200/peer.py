"""The ranks' partial sums added over NVLink by this library's own kernel (fb_peer_reduce_add) instead of an NCCL
all-reduce plus an adding kernel: every rank's partials live in memory that all ranks map (torch's symmetric memory: one
allocation and one rendezvous per process group, plumbing only), and a call is one kernel per rank.

The reference drives one chip (ferrite/runtime.py:304-311) and has no counterpart; llama.added uses this where the
tensor-parallel block adds o_proj's / down_proj's / the experts' partial results back to the residual stream."""
import ctypes

import torch

from . import ops
from ._lib import check, lib

FLAG_BYTES = 1024  # each rank's flag words (one per rank, uint32) at the head of its share of the mapped buffer


class PeerReduce:
    """sites x count bf16 staging buffers per rank (a site: one all-reduce of a decode step, so that a partial is never
    overwritten while another rank may still read the step before's: there is always a later call in between)."""

    def __init__(self, rt, group, count, sites):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        assert sites >= 2, "two staging buffers at least: a rank may refill one while another still reads the call before's"
        self.rt, self.group, self.count, self.sites = rt, group, count, sites
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = FLAG_BYTES + sites * count * 2
        self.mem = symm.empty(nbytes, dtype=torch.uint8, device=rt.device)
        self.mem.zero_()
        self.handle = symm.rendezvous(self.mem, group)
        torch.cuda.synchronize(rt.device)
        dist.barrier(group)  # every rank's flags are zero before anyone signals
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.state = torch.zeros(4, dtype=torch.int32, device=rt.device)
        self.flags = (ctypes.c_void_p * self.world)(*self.bases)
        self.next_site = 0

    def stage(self, rows, cols):
        """Where this rank's next partial goes: a bf16 [1, rows, cols] view of its own staging buffer of the next site."""
        assert rows * cols <= self.count and self.next_site < self.sites, "more all-reduces in a step, or larger, than planned"
        first = FLAG_BYTES + self.next_site * self.count * 2
        return self.mem[first:first + rows * cols * 2].view(torch.bfloat16).view(1, rows, cols)

    def reduce_add(self, n, residual, out):
        """out = residual + every rank's staged partial of the current site (n values each); moves on to the next site."""
        first = FLAG_BYTES + self.next_site * self.count * 2
        partials = (ctypes.c_void_p * self.world)(*[b + first for b in self.bases])
        check(lib().fb_peer_reduce_add(partials, self.flags, self.rank, self.world, self.state.data_ptr(), n,
                                       residual.data_ptr() if residual is not None else None, out.data_ptr(), ops._stream()))
        ops.count()
        self.next_site += 1

    def selftest(self):
        """Three small reductions of known values; raises if a rank does not arrive or a sum is wrong.  Collective."""
        n = min(self.count, 4096)
        out = torch.empty(n, dtype=torch.bfloat16, device=self.rt.device)
        for i in range(3):
            # (sites in turn: a rank leaves call i once every rank has entered it, not finished reading - it must not
            # refill the buffer a slower rank is still adding up)
            self.next_site = i % 2
            self.stage(1, n).fill_(float(self.rank + 1 + i))
            self.reduce_add(n, None, out)
            torch.cuda.synchronize(self.rt.device)
            self.check()
            want = float(sum(r + 1 + i for r in range(self.world)))
            assert bool((out.float() == want).all()), f"fb_peer_reduce_add gave {out[:4].tolist()} for {want}"
        self.new_step()

    def new_step(self):
        self.next_site = 0

    def check(self):
        """After a synchronise: raise if a bounded wait for a rank gave up (the kernel records which)."""
        code = int(self.state[2].item())
        if code:
            self.state[2] = 0
            raise TimeoutError(f"fb_peer_reduce_add: rank {code - 201} did not arrive within the wait's bound")
