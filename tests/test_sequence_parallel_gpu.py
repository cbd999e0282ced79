"""The sequence-parallel path on real GPUs: two ranks over NCCL, each with half of the
positions, against the fp64 oracle of the whole sequence.  Needs two GPUs; skipped otherwise."""
import os
import socket
import sys
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, dtype_name, errq, peer_exchange=False):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist
        from oracle import causal_oracle as orc
        import fast_transformers_b200 as ftb
        from fast_transformers_b200 import sequence_parallel as sp
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        dtype = getattr(torch, dtype_name)
        D = 128 if dtype == torch.bfloat16 else 64
        g = torch.Generator().manual_seed(31)
        N, H, L = 1, 3, 1024 * world
        Q, K = (torch.nn.functional.elu(torch.randn(N, H, L, D, generator=g)) + 1 for _ in range(2))
        V, G = (torch.randn(N, H, L, D, generator=g) for _ in range(2))
        Q, K, V, G = (t.to(dtype) for t in (Q, K, V, G))
        want = (orc.chunked_forward(Q.float(), K.float(), V.float()),) + tuple(
            orc.chunked_backward(Q.float(), K.float(), V.float(), G.float()))
        q, k, v = (sp.shard_sequence(t, rank, world).cuda().requires_grad_(True) for t in (Q, K, V))
        exchange = sp.PeerExchange((N, H, D, D)) if peer_exchange else None
        with ftb.mode(mode):
            for _ in range(3 if peer_exchange else 1):     # the slots alternate: use both twice
                q.grad = k.grad = v.grad = None
                out = sp.sequence_parallel_causal_dot_product(q, k, v, exchange=exchange)
                out.backward(sp.shard_sequence(G, rank, world).cuda())
        torch.cuda.synchronize()
        if exchange is not None:
            exchange.check()
        tol = 1e-5 if (mode == "fp32" and dtype == torch.float32) else 2e-2
        for name, a, b in zip(("out", "gQ", "gK", "gV"), (out, q.grad, k.grad, v.grad), want):
            # error relative to the largest magnitude of the WHOLE tensor, as everywhere else
            ref = sp.shard_sequence(b, rank, world)
            err = (a.double().cpu() - ref).abs().max().item() / b.abs().max().item()
            assert err < tol, "%s rank %d: %.3e" % (name, rank, err)
        if exchange is not None:
            exchange.close()
        dist.destroy_process_group()
    except Exception:
        errq.put("rank %d: %s" % (rank, traceback.format_exc()))


def test_two_ranks_peer_exchange():
    """The same split with the states exchanged through peer memory (``PeerExchange``: partial
    sums pushed into the peers' buffers, a bounded wait on the receiving side) instead of
    ``all_gather``; three steps in a row, so both slots of every source are reused."""
    _run_two_ranks("mma", "bfloat16", True)


@pytest.mark.parametrize("mode,dtype_name", [("fp32", "float32"), ("mma", "float32"), ("mma", "bfloat16")])
def test_two_ranks_match_whole_sequence(mode, dtype_name):
    _run_two_ranks(mode, dtype_name, False)


def _run_two_ranks(mode, dtype_name, peer_exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, dtype_name, errq, peer_exchange))
             for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    assert not alive, "ranks hung"
    assert not errors, "\n".join(errors)
