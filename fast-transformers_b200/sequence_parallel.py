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

``PeerExchange`` is the same exclusive prefix / suffix without a library collective: the ranks
of one node store their states into each other's buffers (peer memory mapped through CUDA IPC)
and a small kernel adds up what has arrived -- two launches per direction, no host
synchronisation, nothing that a CUDA graph cannot hold.  Pass it as ``exchange=``.
"""
import ctypes

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

    def state_parts(self, x, y, reverse=False):
        """Like ``state_sum`` but without adding the partial sums up: returns
        ``(parts, blocks_per_pair, token)`` -- ``parts`` a float32 view of the workspace holding
        ``blocks_per_pair`` (D, M) blocks per (batch, head) pair -- or None when this shape and mode
        keep no raw partial sums.  ``PeerExchange.push_parts`` adds them up while it sends them."""
        from .causal_product import causal_state_parts
        total = self._bytes(x, y, reverse)
        ws = torch.empty(max(total, 1), dtype=torch.uint8, device=x.device)
        half = ws[total // 2:] if reverse else ws
        n = causal_state_parts(x, y, half, mode=self.mode)
        if n == 0:
            return None
        N, H, _, D = x.shape
        count = N * H * n * D * y.shape[3]
        return half[:4 * count].view(torch.float32), n, ws

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

    # The backward in two calls: grad_Q reads the forward states only, so it can run while the
    # reverse states of the other ranks are still on their way.
    def backward_queries(self, Q, K, V, G, initial_state, fwd_token, bwd_token):
        from .causal_product import causal_dot_backward_cuda
        gq = torch.empty_like(Q)
        use_fwd = fwd_token if (fwd_token is not None and self.mode == "mma") else None
        causal_dot_backward_cuda(Q, K, V, G, gq, None, None, self.mode, initial_state=initial_state,
                                 forward_workspace=use_fwd, workspace=bwd_token,
                                 workspace_has_grad_states=True)
        return gq

    def backward_keys_values(self, Q, K, V, G, initial_grad_state, bwd_token):
        from .causal_product import causal_dot_backward_cuda
        gk, gv = torch.empty_like(K), torch.empty_like(V)
        causal_dot_backward_cuda(Q, K, V, G, None, gk, gv, self.mode,
                                 initial_grad_state=initial_grad_state, workspace=bwd_token,
                                 workspace_has_grad_states=True)
        return gk, gv


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


class PeerExchange(object):
    """``exclusive_scan_over_ranks`` for states of one fixed shape, over peer memory instead of
    ``all_gather``: ``ftb_exchange_push`` + ``ftb_exchange_receive`` on the current stream.

    All ranks of ``group`` must be processes of ONE node, each on a GPU of its own, and must
    construct, use (same order of calls) and ``close`` the object together; construction and
    ``close`` contain host collectives (the exchange of the buffers' IPC handles, barriers).
    A rank that never delivers makes the others' receive give up after about a second
    (``ftb_exchange_wait_limit_ms``): the result is then NaN and ``ftb_device_status`` reports the
    timeout.  The kernels cannot raise, so call ``check()`` (it synchronises the device) before a
    step's results are trusted -- once per step, or once per timed region in a benchmark."""

    def __init__(self, state_shape, group=None, device=None):
        from . import _native
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self._lib = _native.lib()
        self._native = _native
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.shape = tuple(int(d) for d in state_shape)
        self.elems = 1
        for d in self.shape:
            self.elems *= d
        self.device = (torch.device(device) if device is not None
                       else torch.device("cuda", torch.cuda.current_device()))
        self._own = ctypes.c_void_p()
        self._peers = [None] * self.world
        handle = ctypes.create_string_buffer(_native.EXCHANGE_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            _native.check(self._lib.ftb_exchange_create(self.world, self.elems,
                                                        ctypes.byref(self._own), handle),
                          "ftb_exchange_create")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self._bufs = (ctypes.c_void_p * self.world)()
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if r == self.rank:
                    self._bufs[r] = self._own.value
                    continue
                ptr = ctypes.c_void_p()
                _native.check(self._lib.ftb_exchange_open(handles[r], ctypes.byref(ptr)),
                              "ftb_exchange_open")
                self._peers[r] = ptr
                self._bufs[r] = ptr.value
        dist.barrier(group=group)      # nobody pushes into a buffer that is not mapped everywhere

    def _stream(self, device):
        return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    def push(self, local, reverse=False):
        """Deliver this rank's state to the ranks after it (before it when ``reverse``)."""
        if self._own is None:
            raise RuntimeError("this exchange has been closed")
        if tuple(local.shape) != self.shape or local.dtype != torch.float32 or not local.is_cuda:
            raise RuntimeError("expected a float32 CUDA state of shape %r" % (self.shape,))
        local = local.contiguous()
        with torch.cuda.device(local.device):
            self._native.check(self._lib.ftb_exchange_push(
                ctypes.c_void_p(local.data_ptr()), self.elems, self._bufs, self.rank, self.world,
                int(bool(reverse)), self._stream(local.device)), "ftb_exchange_push")

    def push_parts(self, parts, blocks_per_unit, reverse=False):
        """The same for a state that exists only as partial sums: ``parts`` is a contiguous float32
        tensor holding, for every unit (a (batch, head) pair: ``shape[0] * shape[1]`` of them),
        ``blocks_per_unit`` blocks whose sum is the unit's state; they are added up on the way."""
        if self._own is None:
            raise RuntimeError("this exchange has been closed")
        units = self.shape[0] * self.shape[1]
        unit_elems = self.elems // max(units, 1)
        if parts.dtype != torch.float32 or not parts.is_cuda or not parts.is_contiguous() or \
                parts.numel() != self.elems * blocks_per_unit:
            raise RuntimeError("parts does not hold %d blocks per unit of a %r state"
                               % (blocks_per_unit, self.shape))
        with torch.cuda.device(parts.device):
            self._native.check(self._lib.ftb_exchange_push_parts(
                ctypes.c_void_p(parts.data_ptr()), unit_elems, int(blocks_per_unit), units, self._bufs,
                self.rank, self.world, int(bool(reverse)), self._stream(parts.device)),
                "ftb_exchange_push_parts")

    def receive(self, reverse=False):
        """Sum of the states delivered by the ranks before this one (after it when ``reverse``);
        zeros when there are none.  Waits (on the GPU, bounded) for the peers' pushes of the same
        exchange; every rank must have issued its own push of that exchange before."""
        if self._own is None:
            raise RuntimeError("this exchange has been closed")
        out = torch.empty(self.shape, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            self._native.check(self._lib.ftb_exchange_receive(
                self._own, ctypes.c_void_p(out.data_ptr()), self.elems, self.rank, self.world,
                int(bool(reverse)), self._stream(self.device)), "ftb_exchange_receive")
        return out

    def exclusive_scan(self, local, reverse=False):
        """Sum of ``local`` over the ranks before this one (after it when ``reverse``)."""
        self.push(local, reverse)
        return self.receive(reverse)

    def check(self):
        """Synchronise this device (all streams) and raise if a push or receive gave up waiting
        for a peer."""
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            self._native.check(self._lib.ftb_device_status(1), "sequence-parallel exchange")

    def close(self):
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)             # every rank is done with every buffer
        with torch.cuda.device(self.device):
            for ptr in self._peers:
                if ptr is not None:
                    self._lib.ftb_exchange_close(ptr)
        dist.barrier(group=self.group)             # every mapping is gone before a buffer is freed
        with torch.cuda.device(self.device):
            self._lib.ftb_exchange_destroy(self._own)
        self._own, self._peers = None, []


def _split_ops(ops, exchange):
    """The peer-memory exchange lets a rank push partial sums and overlap the wait for its peers
    with work that does not need them; it is used when the local operations offer the pieces."""
    return exchange is not None and all(hasattr(ops, n) for n in (
        "state_parts", "backward_queries", "backward_keys_values")) and \
        hasattr(exchange, "push_parts")


class SequenceParallelCausalDotProduct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, group, ops, exchange):
        pushed = False
        if _split_ops(ops, exchange):
            got = ops.state_parts(K.detach(), V.detach(), reverse=False)
            if got is not None:
                parts, n, token = got
                exchange.push_parts(parts, n, reverse=False)
                S_init = exchange.receive(reverse=False)
                pushed = True
        if not pushed:
            T, token = ops.state_sum(K.detach(), V.detach(), reverse=False)
            S_init = (exchange.exclusive_scan(T, reverse=False) if exchange is not None
                      else exclusive_scan_over_ranks(T, group, reverse=False))
        out = ops.forward(Q.detach(), K.detach(), V.detach(), S_init, token)
        ctx.save_for_backward(Q, K, V, S_init)
        ctx.group, ctx.ops, ctx.token, ctx.exchange = group, ops, token, exchange
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, S_init = ctx.saved_tensors
        ops, exchange = ctx.ops, ctx.exchange
        G = grad_out if grad_out.dtype == Q.dtype else grad_out.to(Q.dtype)
        if _split_ops(ops, exchange):
            got = ops.state_parts(Q.detach(), G, reverse=True)
            if got is not None:
                # push the reverse partial sums, compute grad_Q (it needs none of the peers'
                # states) while they travel, then receive and finish
                parts, n, bwd_token = got
                exchange.push_parts(parts, n, reverse=True)
                gq = ops.backward_queries(Q.detach(), K.detach(), V.detach(), G, S_init, ctx.token, bwd_token)
                R_init = exchange.receive(reverse=True)
                gk, gv = ops.backward_keys_values(Q.detach(), K.detach(), V.detach(), G, R_init, bwd_token)
                return gq, gk, gv, None, None, None
        U, bwd_token = ops.state_sum(Q.detach(), G, reverse=True)
        R_init = (exchange.exclusive_scan(U, reverse=True) if exchange is not None
                  else exclusive_scan_over_ranks(U, ctx.group, reverse=True))
        gq, gk, gv = ops.backward(Q.detach(), K.detach(), V.detach(), G, S_init, R_init,
                                  ctx.token, bwd_token)
        return gq, gk, gv, None, None, None


def sequence_parallel_causal_dot_product(Q, K, V, group=None, ops=None, exchange=None):
    """``causal_dot_product`` for this rank's slice (N, H, L/P, dim) of a sequence split in rank
    order over ``group``.  Every rank must call it (it contains collectives), in forward and in
    backward.  Errors of the collectives (a rank that never joins: the process group's timeout)
    surface as exceptions on the host; no kernel waits on another rank -- unless ``exchange`` is a
    ``PeerExchange`` (states of shape (N, H, D, M)), whose receive kernel waits, bounded, for the
    peers' stores instead of the collective."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    return SequenceParallelCausalDotProduct.apply(Q, K, V, group, ops or LocalOps(), exchange)


def shard_sequence(t, rank, world, dim=2):
    """This rank's contiguous slice of the position axis (positions must divide evenly)."""
    L = t.shape[dim]
    if L % world:
        raise ValueError("sequence length %d is not divisible by %d ranks" % (L, world))
    step = L // world
    return t.narrow(dim, rank * step, step)
