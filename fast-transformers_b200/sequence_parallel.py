"""Causal dot product with the SEQUENCE split across ranks (one process per GPU).

Rank r of P holds the positions [r*L/P, (r+1)*L/P) of every (batch, head) pair.  The running
state is additive, so one exchange per direction is enough:

    forward :  T_r = K_r^T V_r                      (local, one pass over K_r, V_r)
               S_init(r) = sum_{r' < r} T_r'         (exclusive prefix over ranks)
               out_r = local pass started from S_init(r)
    backward:  U_r = Q_r^T G_r
               R_init(r) = sum_{r' > r} U_r'         (exclusive suffix over ranks)
               grads_r = local backward started from S_init(r) and R_init(r)

The exchanged message is one fp32 (N, H, D, M) state per rank (1 MiB for H=16, D=M=128), moved
with ``all_gather`` -- NCCL over NVLink on GPUs, gloo in the CPU tests -- and reduced locally
(the gathered states land in this rank's own memory before any kernel reads them).  The
reference is single-device and has no counterpart; the recurrence that is being split is
``fast_transformers/causal_product/causal_product_cpu.cpp:106-121,165-206``.

The three local operations are injectable so the host logic (which rank adds what, autograd
wiring, failure behaviour) can be exercised without a GPU.
"""
import torch
import torch.distributed as dist


class LocalOps(object):
    """The three per-rank operations.  The default implementation is the native library.

    ``state_sum`` returns the rank-local total and a token (the workspace holding the
    per-segment states it computed on the way); ``forward`` / ``backward`` take the tokens back so
    K, V (and Q, grad_out) are swept once, not twice."""

    def __init__(self, mode=None):
        from .settings import get_mode
        self.mode = mode or get_mode()

    def _bytes(self, Q, V, backward):
        from .causal_product import workspace_bytes
        N, H, L, D = Q.shape
        return workspace_bytes(N, H, L, D, V.shape[3], Q.dtype, self.mode, backward=backward,
                               want_state=True)

    def state_sum(self, x, y, reverse=False):
        from .causal_product import causal_state_sum
        if not reverse:
            ws = torch.empty(max(self._bytes(x, y, False), 1), dtype=torch.uint8, device=x.device)
            return causal_state_sum(x, y, mode=self.mode, workspace=ws), ws
        # the backward's workspace: [forward-state half | grad-state half]
        total = self._bytes(x, y, True)
        ws = torch.empty(max(total, 1), dtype=torch.uint8, device=x.device)
        half = ws[total // 2:]
        return causal_state_sum(x, y, mode=self.mode, workspace=half, reverse=True), ws

    def forward(self, Q, K, V, initial_state, token):
        from .causal_product import causal_dot_product_cuda
        out = torch.empty(Q.shape[0], Q.shape[1], Q.shape[2], V.shape[3], device=Q.device,
                          dtype=Q.dtype)
        causal_dot_product_cuda(Q, K, V, out, self.mode, initial_state=initial_state,
                                workspace=token, workspace_has_states=True)
        return out

    def backward(self, Q, K, V, G, initial_state, initial_grad_state, fwd_token, bwd_token):
        from .causal_product import causal_dot_backward_cuda
        gq, gk, gv = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
        use_fwd = fwd_token if (fwd_token is not None and self.mode == "mma") else None
        causal_dot_backward_cuda(Q, K, V, G, gq, gk, gv, self.mode, initial_state=initial_state,
                                 initial_grad_state=initial_grad_state, forward_workspace=use_fwd,
                                 workspace=bwd_token, workspace_has_grad_states=True)
        return gq, gk, gv


def exclusive_scan_over_ranks(local, group=None, reverse=False):
    """Sum of ``local`` over the ranks before this one (after it when ``reverse``); zeros on the
    first (last) rank.  One all_gather of ``local`` plus a local reduction."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return torch.zeros_like(local)
    local = local.contiguous()
    flat = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.reshape(-1), group=group)
    gathered = flat.view((world,) + tuple(local.shape))
    part = gathered[rank + 1:] if reverse else gathered[:rank]
    if part.shape[0] == 0:
        return torch.zeros_like(local)
    return part.sum(dim=0)


class SequenceParallelCausalDotProduct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, group, ops):
        T, token = ops.state_sum(K.detach(), V.detach(), reverse=False)
        S_init = exclusive_scan_over_ranks(T, group, reverse=False)
        out = ops.forward(Q.detach(), K.detach(), V.detach(), S_init, token)
        ctx.save_for_backward(Q, K, V, S_init)
        ctx.group, ctx.ops, ctx.token = group, ops, token
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, S_init = ctx.saved_tensors
        G = grad_out if grad_out.dtype == Q.dtype else grad_out.to(Q.dtype)
        U, bwd_token = ctx.ops.state_sum(Q.detach(), G, reverse=True)
        R_init = exclusive_scan_over_ranks(U, ctx.group, reverse=True)
        gq, gk, gv = ctx.ops.backward(Q.detach(), K.detach(), V.detach(), G, S_init, R_init,
                                      ctx.token, bwd_token)
        return gq, gk, gv, None, None


def sequence_parallel_causal_dot_product(Q, K, V, group=None, ops=None):
    """``causal_dot_product`` for this rank's slice (N, H, L/P, dim) of a sequence split in rank
    order over ``group``.  Every rank must call it (it contains collectives), in forward and in
    backward.  Errors of the collectives (a rank that never joins: the process group's timeout)
    surface as exceptions on the host; no kernel waits on another rank."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    return SequenceParallelCausalDotProduct.apply(Q, K, V, group, ops or LocalOps())


def shard_sequence(t, rank, world, dim=2):
    """This rank's contiguous slice of the position axis (positions must divide evenly)."""
    L = t.shape[dim]
    if L % world:
        raise ValueError("sequence length %d is not divisible by %d ranks" % (L, world))
    step = L // world
    return t.narrow(dim, rank * step, step)
