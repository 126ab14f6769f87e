"""Context parallelism across GPUs for one long sequence (per-channel and scalar gate alike).

Rank r owns the r-th contiguous, chunk-aligned slice of the sequence.  The recurrence is affine in the state,
S_out = M S_in + H, so one exchange per pass is enough:

  forward   every rank runs the state + transition pre-pass over its own segments, folds them into one rank-level pair
            (H_r, M_r), all-gathers the pairs (fp32, 2 x HV x 64 KiB per rank) into local memory and left-folds the
            ranks before it, in rank order, to obtain the state entering its slice;
  backward  the same with (D_r, M_r^T) folded from the ranks after it.

This is the mechanism the reference has for the scalar gate only (mogan_kda/ops/gated_delta_rule/chunk/cp/preprocess.py:37-90,
cp/comm.py:14-43: one ``all_gather_into_tensor`` of packed (h, M) per pass); here M is the full K x K per-channel
transition.  Rank r consumes only ranks < r in the forward pass, in index order, so the result does not depend on how
many ranks follow.  The collective is NCCL's all-gather into this GPU's own memory; no kernel reads a peer's memory.
"""
import torch
import torch.distributed as dist

from . import ops


class ContextParallel:
    """Pass as ``cp_context=`` to ``chunk_kda`` / ``chunk_delta_rule`` / ``chunk_gated_delta_rule``; each rank calls with
    its own slice (B == 1, slice length a multiple of 64 on every rank but the last)."""

    is_inter = True

    def __init__(self, group=None, *, comm=None):
        """``group``: a torch.distributed process group (default: WORLD).  ``comm`` (tests): any object with ``rank``,
        ``world`` and ``all_gather(flat_out, flat_in)`` replacing the process group."""
        self.comm = comm
        if comm is not None:
            self.group, self.rank, self.world = None, comm.rank, comm.world
        else:
            self.group = group if group is not None else dist.group.WORLD
            self.rank = dist.get_rank(self.group)
            self.world = dist.get_world_size(self.group)
        self._m_rank = None

    # -- plumbing -----------------------------------------------------------------------------------------------
    def _gather_pairs(self, a, m):
        """all-gather (a, m) [1,HV,K,K] each -> ([W,HV,K,K], [W,HV,K,K])."""
        mine = torch.stack([a[0], m[0]]).contiguous()
        flat = torch.empty(self.world * mine.numel(), dtype=mine.dtype, device=mine.device)
        if self.comm is not None:
            self.comm.all_gather(flat, mine.view(-1))
        else:
            dist.all_gather_into_tensor(flat, mine.view(-1), group=self.group)
        out = flat.view((self.world,) + tuple(mine.shape))
        return out[:, 0].contiguous(), out[:, 1].contiguous()

    def _rank_offsets(self, device):
        return torch.tensor([0, self.world], dtype=torch.int32, device=device)

    # -- hooks called by the autograd function ------------------------------------------------------------------------
    def forward_carry(self, hs, ms, carry, lay, HV):
        """hs, ms [NS,HV,K,K]: per local segment (state reached from zero, transition).  ``carry`` = the caller's
        initial state ([1,HV,K,V], meaningful on rank 0 only).  Returns the state entering this rank's slice."""
        if lay.NG != 1:
            raise ValueError("cross-GPU context parallelism handles one sequence per call")
        first = self.rank == 0
        _, h_rank = ops.state_combine(lay.grp_seg_off, 1, lay.NS, HV, hs, ms, carry=carry if first else None, want_in=False)
        eye = torch.eye(ms.shape[-1], dtype=ms.dtype, device=ms.device).expand(1, HV, -1, -1).contiguous()
        _, m_rank = ops.state_combine(lay.grp_seg_off, 1, lay.NS, HV, None, ms, carry=eye, want_in=False)
        self._m_rank = m_rank
        if self.world == 1:
            return carry
        all_h, all_m = self._gather_pairs(h_rank, m_rank)
        s_in, _ = ops.state_combine(self._rank_offsets(ms.device), 1, self.world, HV, all_h, all_m, want_out=False)
        return carry if first else s_in[self.rank:self.rank + 1].contiguous()

    def backward_carry(self, dloc, ms, carry, lay, HV):
        """dloc [NS,HV,K,K]: per local segment, gradient of the state entering it given zero from the right.
        ``carry`` = gradient of the final state (meaningful on the last rank only).  Returns the gradient of the state
        leaving this rank's slice."""
        last = self.rank == self.world - 1
        if self.world == 1:
            return carry
        _, d_rank = ops.state_combine(lay.grp_seg_off, 1, lay.NS, HV, dloc, ms, carry=carry if last else None, reverse=True,
                                      want_in=False)
        all_d, all_m = self._gather_pairs(d_rank, self._m_rank)
        g_in, _ = ops.state_combine(self._rank_offsets(ms.device), 1, self.world, HV, all_d, all_m, reverse=True, want_out=False)
        return carry if last else g_in[self.rank:self.rank + 1].contiguous()

    def finish_backward(self, dh0):
        """Gradient w.r.t. the state entering this rank's slice; the caller's initial state lives on rank 0."""
        return dh0
