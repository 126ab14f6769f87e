"""Context parallelism across GPUs (per-channel and scalar gate alike): one long sequence, or a packed batch of
sequences, is cut into equal contiguous token slices, one per rank.

Rank r owns the r-th slice.  A sequence may start on one rank and end on a later one; sequences that lie inside a
slice are local.  The recurrence is affine in the state, S_out = M S_in + H, so one exchange per pass is enough:

  forward   every rank runs the state + transition pre-pass over its own segments, folds those of its LAST local
            sequence into one pair (H_r, M_r), all-gathers the pairs (fp32, 2 x HV x 64 KiB per rank) into local
            memory and left-folds the ranks that hold earlier parts of its FIRST local sequence, in rank order, to
            obtain the state entering its slice;
  backward  the same with (D_r, M_r^T) of the first local sequence, folded from the ranks that hold later parts of
            the last local sequence.

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
    its own token slice (B == 1).

    Without a topology (``ContextParallel(group)``) the whole call is ONE sequence spanning every rank.  With the
    topology of a packed batch (``build_cp_context``) the context carries this rank's local ``cu_seqlens`` and the
    number of ranks before / after it that share its first / last local sequence; the fields have the names of the
    reference's context (mogan_kda/ops/gated_delta_rule/chunk/cp/context.py:27-50)."""

    is_inter = True

    def __init__(self, group=None, *, comm=None, cu_seqlens=None, cu_seqlens_cpu=None, pre_num_ranks=None,
                 post_num_ranks=None, conv1d_kernel_size=None, pre_num_conv_tokens=None):
        """``group``: a torch.distributed process group (default: WORLD).  ``comm`` (tests): any object with ``rank``,
        ``world`` and ``all_gather(flat_out, flat_in)`` replacing the process group."""
        self.comm = comm
        if comm is not None:
            self.group, self.rank, self.world = None, comm.rank, comm.world
        else:
            self.group = group if group is not None else dist.group.WORLD
            self.rank = dist.get_rank(self.group)
            self.world = dist.get_world_size(self.group)
        self.cu_seqlens, self.cu_seqlens_cpu = cu_seqlens, cu_seqlens_cpu
        self.pre_num_ranks = self.rank if pre_num_ranks is None else int(pre_num_ranks)
        self.post_num_ranks = self.world - 1 - self.rank if post_num_ranks is None else int(post_num_ranks)
        if not (0 <= self.pre_num_ranks <= self.rank and 0 <= self.post_num_ranks <= self.world - 1 - self.rank):
            raise ValueError("pre_num_ranks / post_num_ranks reach outside the group")
        self.is_first_rank, self.is_last_rank = self.pre_num_ranks == 0, self.post_num_ranks == 0
        self.conv1d_kernel_size, self.pre_num_conv_tokens = conv1d_kernel_size, pre_num_conv_tokens

    @property
    def num_seqs(self):
        return 0 if self.cu_seqlens is None else self.cu_seqlens.numel() - 1

    @property
    def conv_halo_tokens(self):
        """Tokens of the previous rank a causal short convolution in front of this op needs for this rank's first
        local sequence: min(kernel - 1, tokens of that sequence that lie before this slice); None without the fields."""
        if self.conv1d_kernel_size is None or self.pre_num_conv_tokens is None:
            return None
        return min(self.conv1d_kernel_size - 1, self.pre_num_conv_tokens)

    # -- plumbing -----------------------------------------------------------------------------------------------
    def _gather_pairs(self, a, m):
        """all-gather (a, m) [HV,K,K] each -> ([W,HV,K,K], [W,HV,K,K])."""
        mine = torch.stack([a, m]).contiguous()
        flat = torch.empty(self.world * mine.numel(), dtype=mine.dtype, device=mine.device)
        if self.comm is not None:
            self.comm.all_gather(flat, mine.view(-1))
        else:
            dist.all_gather_into_tensor(flat, mine.view(-1), group=self.group)
        out = flat.view((self.world,) + tuple(mine.shape))
        return out[:, 0], out[:, 1]

    @staticmethod
    def _fold(h, m, HV, reverse):
        """Left fold (reverse: right fold) of n rank-level pairs from zero -> [1,HV,K,K]."""
        n = h.shape[0]
        off = torch.tensor([0, n], dtype=torch.int32, device=m.device)
        _, out = ops.state_combine(off, 1, n, HV, h.contiguous(), m.contiguous(), reverse=reverse, want_in=False)
        return out

    # -- hooks called by the autograd function ------------------------------------------------------------------------
    def forward_carry(self, hs, ms, carry, lay, HV):
        """hs, ms [NS,HV,K,K]: per local segment (state reached from zero, transition).  ``carry`` = the caller's
        initial states of the local sequences ([NG,HV,K,V] or None); its first row is ignored unless the first local
        sequence starts on this rank.  Returns ``(states entering the local sequences, m_first)``; ``m_first`` is the
        transition of the first local sequence over this rank's slice, which the backward exchange sends to the earlier
        ranks.  It belongs to this call, not to the context (one context serves every layer of a model): the caller keeps
        it with its saved tensors and hands it to ``backward_carry``."""
        NG, K = lay.NG, ms.shape[-1]
        if carry is not None and not self.is_first_rank:
            carry = carry.clone()
            carry[0] = 0
        _, h_all = ops.state_combine(lay.grp_seg_off, NG, lay.NS, HV, hs, ms, carry=carry, want_in=False)
        eye = torch.eye(K, dtype=ms.dtype, device=ms.device).expand(NG, HV, K, K).contiguous()
        _, m_all = ops.state_combine(lay.grp_seg_off, NG, lay.NS, HV, None, ms, carry=eye, want_in=False)
        m_first = m_all[0].clone()
        if self.world == 1:
            return carry, m_first
        all_h, all_m = self._gather_pairs(h_all[NG - 1], m_all[NG - 1])       # every rank joins the collective
        if self.is_first_rank:
            return carry, m_first
        lo = self.rank - self.pre_num_ranks
        s_in = self._fold(all_h[lo:self.rank], all_m[lo:self.rank], HV, False)
        out = carry if carry is not None else torch.zeros(NG, HV, K, K, dtype=ms.dtype, device=ms.device)
        out[0] = s_in[0]
        return out, m_first

    def backward_carry(self, dloc, ms, carry, lay, HV, m_first):
        """dloc [NS,HV,K,K]: per local segment, gradient of the state entering it given zero from the right.
        ``carry`` = gradients of the local sequences' final states ([NG,HV,K,V] or None); its last row is ignored unless
        the last local sequence ends on this rank.  ``m_first``: what ``forward_carry`` returned for the same call.
        Returns the gradients of the states leaving the local sequences."""
        NG, K = lay.NG, ms.shape[-1]
        if self.world == 1:
            return carry
        if carry is not None and not self.is_last_rank:
            carry = carry.clone()
            carry[NG - 1] = 0
        _, d_all = ops.state_combine(lay.grp_seg_off, NG, lay.NS, HV, dloc, ms, carry=carry, reverse=True, want_in=False)
        all_d, all_m = self._gather_pairs(d_all[0], m_first)
        if self.is_last_rank:
            return carry
        lo, hi = self.rank + 1, self.rank + 1 + self.post_num_ranks
        g_in = self._fold(all_d[lo:hi], all_m[lo:hi], HV, True)
        out = carry if carry is not None else torch.zeros(NG, HV, K, K, dtype=ms.dtype, device=ms.device)
        out[NG - 1] = g_in[0]
        return out

    def finish_backward(self, dh0):
        """Gradient w.r.t. the caller's initial states.  The state entering a sequence that started on an earlier rank is
        not this rank's input: its row is zero (mogan_kda/ops/gated_delta_rule/chunk/__init__.py:178-186)."""
        if dh0 is not None and not self.is_first_rank:
            dh0 = dh0.clone()
            dh0[0] = 0
        return dh0


def partition_tokens(cu_seqlens, world, rank):
    """Host arithmetic of the equal-token split of a packed batch (restated from ``_calc_inter_cp_seqs``,
    mogan_kda/ops/gated_delta_rule/chunk/cp/context.py:182-243).  ``cu_seqlens``: the GLOBAL boundaries as a list or a
    CPU tensor.  Returns a dict: ``rank_start``, ``rank_end``, ``cu_seqlens`` (local boundaries, list),
    ``pre_num_ranks`` / ``post_num_ranks`` (ranks before / after this one that hold part of its first / last local
    sequence), ``is_first_rank`` / ``is_last_rank`` and ``pre_num_conv_tokens`` (tokens of the first local sequence that
    lie before the slice)."""
    cu = [int(x) for x in (cu_seqlens.tolist() if hasattr(cu_seqlens, "tolist") else cu_seqlens)]
    total = cu[-1]
    if total % world != 0:
        raise AssertionError(f"inter-card CP requires total tokens ({total}) divisible by world_size ({world}); "
                             "pad/reshape the global sequence to a multiple of world_size.")
    part = total // world
    a, b = part * rank, part * (rank + 1)
    # sequences that overlap [a, b): first = the one containing token a, last = the one containing token b - 1
    first = 0
    while cu[first + 1] <= a:
        first += 1
    last = first
    while cu[last + 1] < b:
        last += 1
    local = sorted({min(max(x, a), b) - a for x in cu[first:last + 2]})
    first_start, last_end = cu[first], cu[last + 1]
    first_rank, last_rank = first_start // part, (last_end - 1) // part
    return dict(rank_start=a, rank_end=b, cu_seqlens=local, pre_num_ranks=rank - first_rank,
                post_num_ranks=last_rank - rank, is_first_rank=rank == first_rank, is_last_rank=rank == last_rank,
                pre_num_conv_tokens=max(0, a - first_start))


def build_cp_context(cu_seqlens, *, group=None, comm=None, conv1d_kernel_size=None, cu_seqlens_cpu=None):
    """Context for a packed batch split into equal token slices over the ranks of ``group`` (the inter-card mode of the
    reference's ``build_cp_context``, mogan_kda/ops/gated_delta_rule/chunk/cp/context.py:108-178).  ``cu_seqlens``
    holds the GLOBAL boundaries (int tensor [N+1]; pass ``cu_seqlens_cpu`` as well to avoid a device read).  The caller
    slices its tensors to tokens [rank_start, rank_end) = rank * total / world ... and passes the returned context as
    ``cp_context=`` (its local ``cu_seqlens`` replaces the ``cu_seqlens`` argument); ``initial_state`` and the final
    state have one row per LOCAL sequence.  Every local sequence is additionally cut into concurrent segments on the
    GPU, which is the combined inter + intra mode."""
    ctx = ContextParallel(group, comm=comm)
    host = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
    part = partition_tokens(host, ctx.world, ctx.rank)
    local = torch.tensor(part["cu_seqlens"], dtype=torch.int32)
    return ContextParallel(group, comm=comm, cu_seqlens=local.to(cu_seqlens.device, non_blocking=True), cu_seqlens_cpu=local,
                           pre_num_ranks=part["pre_num_ranks"], post_num_ranks=part["post_num_ranks"],
                           conv1d_kernel_size=conv1d_kernel_size, pre_num_conv_tokens=part["pre_num_conv_tokens"])
