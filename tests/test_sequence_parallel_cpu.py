"""Host logic of the sequence-parallel path on CPU ranks (gloo): which rank adds which states,
autograd wiring, and the failure path (a rank that never joins ends the others' collective
with an error after the process-group timeout).  The per-rank kernels are replaced by the CPU
oracle; the GPU path itself is covered by the ``gpu``-marked tests."""
import datetime
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class OracleOps(object):
    """fp64 stand-ins for the three local operations."""

    def state_sum(self, x, y, reverse=False):
        from oracle import causal_oracle as orc
        return orc.local_states(None, x, y), None

    def forward(self, Q, K, V, initial_state, token):
        from oracle import causal_oracle as orc
        return orc.chunked_forward(Q, K, V, chunk=16, initial_state=initial_state)

    def backward(self, Q, K, V, G, initial_state, initial_grad_state, fwd_token, bwd_token):
        from oracle import causal_oracle as orc
        return orc.chunked_backward(Q, K, V, G, chunk=16, initial_state=initial_state,
                                    final_grad_state=initial_grad_state)


class SplitOracleOps(OracleOps):
    """The pieces the peer-memory path uses: partial sums (here three unequal slices of the
    positions per (batch, head) pair) and the backward in two calls."""

    def state_parts(self, x, y, reverse=False):
        L = x.shape[2]
        cuts = [0, L // 4, L // 2 + 1, L]
        blocks = [(x[:, :, a:b].transpose(-1, -2) @ y[:, :, a:b]) for a, b in zip(cuts, cuts[1:])]
        parts = torch.stack(blocks, dim=2).contiguous()      # (N, H, 3, D, M)
        return parts.reshape(-1), 3, None

    def backward_queries(self, Q, K, V, G, initial_state, fwd_token, bwd_token):
        return self.backward(Q, K, V, G, initial_state, None, None, None)[0]

    def backward_keys_values(self, Q, K, V, G, initial_grad_state, bwd_token):
        return self.backward(Q, K, V, G, None, initial_grad_state, None, None)[1:]


class GlooExchange(object):
    """Stand-in for ``PeerExchange`` with the same push / receive split, over gloo."""

    def __init__(self, shape):
        self.shape, self.pending, self.log = tuple(shape), None, []

    def push_parts(self, parts, blocks_per_unit, reverse=False):
        N, H, D, M = self.shape
        self.push(parts.view(N, H, blocks_per_unit, D, M).sum(dim=2), reverse)

    def push(self, local, reverse=False):
        assert self.pending is None, "two pushes without a receive in between"
        self.pending = (local.contiguous(), reverse)
        self.log.append("push")

    def receive(self, reverse=False):
        from fast_transformers_b200 import sequence_parallel as sp
        local, rev = self.pending
        assert rev == reverse
        self.pending = None
        self.log.append("receive")
        return sp.exclusive_scan_over_ranks(local, reverse=reverse)

    def exclusive_scan(self, local, reverse=False):
        self.push(local, reverse)
        return self.receive(reverse)


def _worker(rank, world, port, case, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        from oracle import causal_oracle as orc
        import fast_transformers_b200  # noqa: F401
        from fast_transformers_b200 import sequence_parallel as sp

        if case == "missing_rank" and rank == world - 1:
            return   # this rank never joins
        timeout = datetime.timedelta(seconds=5 if case == "missing_rank" else 60)
        if case == "missing_rank":
            try:
                dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timeout)
                t = torch.zeros(4, dtype=torch.float64)
                sp.exclusive_scan_over_ranks(t)
            except Exception:
                return   # the expected outcome: an error on the host, nothing hangs
            raise AssertionError("a collective completed although a rank never joined")

        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timeout)
        g = torch.Generator().manual_seed(7)
        N, H, L, D, M = 2, 2, 24 * world, 5, 7
        Q, K, V, G = (torch.rand(N, H, L, d, generator=g, dtype=torch.float64) for d in (D, D, M, M))
        want_out = orc.chunked_forward(Q, K, V, chunk=16)
        want_g = orc.chunked_backward(Q, K, V, G, chunk=16)

        q, k, v = (sp.shard_sequence(t, rank, world).clone().requires_grad_(True) for t in (Q, K, V))
        if case == "split_exchange":
            # the path of the peer-memory exchange: partial sums pushed, grad_Q between the push
            # and the receive of the reverse states
            exchange = GlooExchange((N, H, D, M))
            out = sp.sequence_parallel_causal_dot_product(q, k, v, ops=SplitOracleOps(), exchange=exchange)
            out.backward(sp.shard_sequence(G, rank, world))
            assert exchange.log == ["push", "receive", "push", "receive"] and exchange.pending is None
        else:
            out = sp.sequence_parallel_causal_dot_product(q, k, v, ops=OracleOps())
            out.backward(sp.shard_sequence(G, rank, world))
        assert torch.allclose(out, sp.shard_sequence(want_out, rank, world), rtol=1e-12, atol=1e-12)
        for got, want in zip((q.grad, k.grad, v.grad), want_g):
            assert torch.allclose(got, sp.shard_sequence(want, rank, world), rtol=1e-12, atol=1e-12)

        # the scan itself: rank r receives the sum over ranks before (after) it
        t = torch.full((3,), float(rank + 1), dtype=torch.float64)
        pre = sp.exclusive_scan_over_ranks(t, reverse=False)
        suf = sp.exclusive_scan_over_ranks(t, reverse=True)
        assert pre[0].item() == sum(range(1, rank + 1))
        assert suf[0].item() == sum(range(rank + 2, world + 1))
        dist.destroy_process_group()
    except Exception:
        errq.put("rank %d: %s" % (rank, traceback.format_exc()))


def _run(world, case):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    assert not alive, "ranks hung"
    assert not errors, "\n".join(errors)
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_matches_single_rank(world):
    _run(world, "split")


def test_split_exchange_path_matches_single_rank():
    _run(3, "split_exchange")


def test_rank_that_never_joins_is_an_error_not_a_hang():
    _run(2, "missing_rank")


def test_shard_sequence_rejects_ragged_split():
    from fast_transformers_b200 import sequence_parallel as sp
    with pytest.raises(ValueError):
        sp.shard_sequence(torch.zeros(1, 1, 10, 2), 0, 3)
