"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout is available (its location: the environment variable
``FAST_TRANSFORMERS_REFERENCE``):

    python oracle/build_ref.py            # compiles the reference CPU extension in place
    python tests/golden/make_golden.py    # writes tests/golden/*.npz

The reference's Python modules for this path are imported from the checkout as they are.
Its top-level ``fast_transformers/attention/__init__.py`` imports every attention flavour
(and through them compiled extensions that are not part of this path), so the two package
objects ``fast_transformers`` and ``fast_transformers.attention`` are created empty with
their ``__path__`` pointing into the checkout, and the compiled
``causal_product_cpu`` module built by ``oracle/build_ref.py`` is registered under its
package-qualified name.  Everything else (``causal_product/__init__.py``,
``attention/causal_linear_attention.py``, ``attention/attention_layer.py``,
``feature_maps``, ``masking.py``, ``attention_registry``, ``events``, ``transformers.py``)
executes unmodified.

All inputs come from seeded CPU generators; the fixtures store inputs and outputs (or, for
the benchmark-sized config 1, only a strided sample of the outputs -- the inputs are
regenerated from the seed by ``fast_transformers_b200.workloads``).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref, causal_oracle  # noqa: E402


def import_reference():
    root = build_ref.reference_root()
    if root is None:
        raise SystemExit("reference checkout not found")
    build_ref.build_reference_ext()
    ext = causal_oracle.reference_ext()
    pkg_dir = os.path.join(root, "fast_transformers")
    ft = types.ModuleType("fast_transformers")
    ft.__path__ = [pkg_dir]
    sys.modules["fast_transformers"] = ft
    att = types.ModuleType("fast_transformers.attention")
    att.__path__ = [os.path.join(pkg_dir, "attention")]
    sys.modules["fast_transformers.attention"] = att
    sys.modules["fast_transformers.causal_product.causal_product_cpu"] = ext
    import fast_transformers.causal_product as cp
    import fast_transformers.attention.causal_linear_attention as cla
    import fast_transformers.attention.attention_layer as al
    import fast_transformers.feature_maps as fm
    import fast_transformers.masking as masking
    import fast_transformers.transformers as tr
    return cp, cla, al, fm, masking, tr


def np_(t):
    return t.detach().cpu().numpy()


def main():
    cp, cla, al, fm, masking, tr = import_reference()
    torch.set_num_threads(1)

    # ---- 1. raw product, odd sizes, U[0,1) inputs (the reference tests' distribution) ----
    g = torch.Generator().manual_seed(101)
    N, H, L, D, M = 2, 3, 70, 19, 33
    Q, K, V, G = (torch.rand(N, H, L, d, generator=g) for d in (D, D, M, M))
    Qr, Kr, Vr = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out = cp.causal_dot_product(Qr, Kr, Vr)
    out.backward(G)
    np.savez_compressed(os.path.join(HERE, "product_small.npz"), Q=np_(Q), K=np_(K), V=np_(V),
                        G=np_(G), out=np_(out), gQ=np_(Qr.grad), gK=np_(Kr.grad),
                        gV=np_(Vr.grad))

    # ---- 2. config 1 (B2 H4 L1024 D=M=64), strided sample of the reference outputs --------
    from fast_transformers_b200 import workloads
    Q, K, V, G = workloads.make_inputs(1)
    Qr, Kr, Vr = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out = cp.causal_dot_product(Qr, Kr, Vr)
    out.backward(G)
    rows = torch.arange(7, 1024, 16)
    np.savez_compressed(os.path.join(HERE, "product_config1_sample.npz"), rows=np_(rows),
                        out=np_(out[:, :, rows]), gQ=np_(Qr.grad[:, :, rows]),
                        gK=np_(Kr.grad[:, :, rows]), gV=np_(Vr.grad[:, :, rows]),
                        checksum=np.array([out.double().sum().item(),
                                           Qr.grad.double().sum().item(),
                                           Kr.grad.double().sum().item(),
                                           Vr.grad.double().sum().item()]))

    # ---- 3. the layer: L == S, L < S, L > S, with key lengths ------------------------------
    layer = {}
    for name, (L, S) in {"eq": (24, 24), "lt": (16, 24), "gt": (24, 16)}.items():
        g = torch.Generator().manual_seed(300 + L + 7 * S)
        N, H, E, Mv = 3, 2, 8, 12
        q = torch.randn(N, L, H, E, generator=g).requires_grad_(True)
        k = torch.randn(N, S, H, E, generator=g).requires_grad_(True)
        v = torch.randn(N, S, H, Mv, generator=g).requires_grad_(True)
        w = torch.randn(N, L, H, Mv, generator=g)
        klen = torch.tensor([S, max(1, S - 5), max(1, S // 2)])
        att = cla.CausalLinearAttention(E)
        y = att(q, k, v, masking.TriangularCausalMask(L), masking.LengthMask(torch.full((N,), L)),
                masking.LengthMask(klen, max_len=S))
        assert y.is_contiguous() and torch.isfinite(y).all()
        vals = dict(q=q, k=k, v=v, w=w, klen=klen, y=y)
        if L <= S:
            # For L > S the reference passes V with S rows to a kernel that walks L rows
            # (causal_linear_attention.py:68-69,98-102): its backward then writes grad_V rows
            # S..L-1 past the end of the buffer.  Only the forward is recorded for that case.
            (y * w).sum().backward()
            vals.update(gq=q.grad, gk=k.grad, gv=v.grad)
        for key, val in vals.items():
            layer[name + "_" + key] = np_(val)
    np.savez_compressed(os.path.join(HERE, "layer.npz"), **layer)

    # ---- 4. Favor feature map with a fixed omega -------------------------------------------
    g = torch.Generator().manual_seed(404)
    E, n_dims = 16, 64
    f = fm.Favor(E, n_dims=n_dims)
    omega = workloads.favor_omega(E, n_dims, g)
    f.omega.copy_(omega)
    x = torch.randn(2, 10, 3, E, generator=g) * 0.5
    np.savez_compressed(os.path.join(HERE, "favor.npz"), omega=np_(omega), x=np_(x),
                        phi=np_(f(x)), elu=np_(fm.elu_feature_map(E)(x)))

    # ---- 5. a two-layer causal-linear encoder built from the reference's own classes -------
    torch.manual_seed(505)
    d_model, heads, dq, dff, nl = 32, 4, 8, 64, 2
    enc = tr.TransformerEncoder(
        [tr.TransformerEncoderLayer(
            al.AttentionLayer(cla.CausalLinearAttention(dq), d_model, heads, d_keys=dq, d_values=dq),
            d_model, dff, 0.0, "relu") for _ in range(nl)],
        torch.nn.LayerNorm(d_model))
    g = torch.Generator().manual_seed(506)
    x = torch.rand(2, 40, d_model, generator=g).requires_grad_(True)
    w = torch.randn(2, 40, d_model, generator=g)
    y = enc(x, attn_mask=masking.TriangularCausalMask(40))
    (y * w).sum().backward()
    blob = {"sd__" + k: np_(v) for k, v in enc.state_dict().items()}
    blob.update(x=np_(x), w=np_(w), y=np_(y), gx=np_(x.grad))
    blob.update({"gp__" + k: np_(p.grad) for k, p in enc.named_parameters()})
    np.savez_compressed(os.path.join(HERE, "encoder.npz"), **blob)

    for f_ in sorted(os.listdir(HERE)):
        if f_.endswith(".npz"):
            print(f_, os.path.getsize(os.path.join(HERE, f_)), "bytes")


def import_reference_recurrent():
    """The reference's RecurrentLinearAttention (recurrent/attention/self_attention/
    linear_attention.py).  The package ``__init__`` files above it import every recurrent
    attention flavour, so they are replaced by empty packages as for ``attention``."""
    import_reference()
    root = build_ref.reference_root()
    pkg_dir = os.path.join(root, "fast_transformers")
    for name, rel in (("recurrent", "recurrent"), ("recurrent.attention", "recurrent/attention"),
                      ("recurrent.attention.self_attention", "recurrent/attention/self_attention")):
        m = types.ModuleType("fast_transformers." + name)
        m.__path__ = [os.path.join(pkg_dir, rel)]
        sys.modules["fast_transformers." + name] = m
    import fast_transformers.recurrent.attention.self_attention.linear_attention as rla
    return rla


def recurrent():
    """``recurrent.npz``: the reference module stepped over a short sequence (inputs, every
    output, the final state), once from an empty state and once from a given one, and the
    reference's own check that the steps reproduce the batch form."""
    rla = import_reference_recurrent()
    import fast_transformers.attention.causal_linear_attention as cla
    import fast_transformers.masking as masking
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(606)
    N, H, E, M, L = 3, 4, 25, 64, 12          # the reference test's E and M
    q, k, v = (torch.rand(N, L, H, d, generator=g) for d in (E, E, M))
    S0, z0 = torch.rand(N, H, E, M, generator=g), torch.rand(N, H, E, generator=g)
    att = rla.RecurrentLinearAttention(E).eval()
    blob = {"q": np_(q), "k": np_(k), "v": np_(v), "S0": np_(S0), "z0": np_(z0)}
    with torch.no_grad():
        for tag, state in (("empty", None), ("given", [S0.clone(), z0.clone()])):
            ys = []
            for i in range(L):
                y, state = att(q[:, i], k[:, i], v[:, i], state)
                ys.append(y)
            blob[tag + "_y"] = np_(torch.stack(ys, 1))
            blob[tag + "_S"] = np_(state[0])
            blob[tag + "_z"] = np_(state[1])
        batch = cla.CausalLinearAttention(E).eval()
        lm = masking.LengthMask(torch.full((N,), L, dtype=torch.long))
        blob["batch_y"] = np_(batch(q, k, v, masking.TriangularCausalMask(L), lm, lm))
    assert np.abs(blob["batch_y"] - blob["empty_y"]).max() < 1e-5   # the reference's own bound
    np.savez_compressed(os.path.join(HERE, "recurrent.npz"), **blob)
    print("recurrent.npz", os.path.getsize(os.path.join(HERE, "recurrent.npz")), "bytes")


def recurrent_encoder():
    """``recurrent_encoder.npz``: the reference's ``RecurrentTransformerEncoder`` (two layers of
    ``RecurrentTransformerEncoderLayer(RecurrentAttentionLayer(RecurrentLinearAttention))``, final
    LayerNorm) stepped over a short sequence: its weights, the inputs, every output and the
    per-layer states after the 7th and after the last position."""
    rla = import_reference_recurrent()
    import fast_transformers.recurrent.attention.self_attention.attention_layer as ral
    import fast_transformers.recurrent.transformers as rtr
    torch.set_num_threads(1)
    torch.manual_seed(707)
    heads, dq, d_model, d_ff, N, L, P = 4, 16, 64, 96, 3, 12, 7
    enc = rtr.RecurrentTransformerEncoder(
        [rtr.RecurrentTransformerEncoderLayer(
            ral.RecurrentAttentionLayer(rla.RecurrentLinearAttention(dq), d_model, heads,
                                        d_keys=dq, d_values=dq),
            d_model, d_ff, dropout=0.0, activation="gelu")
         for _ in range(2)],
        torch.nn.LayerNorm(d_model)).eval()
    x = torch.randn(N, L, d_model, generator=torch.Generator().manual_seed(708))
    blob = {"sd__" + k: np_(v) for k, v in enc.state_dict().items()}
    blob["x"] = np_(x)
    with torch.no_grad():
        state, ys = None, []
        for i in range(L):
            y, state = enc(x[:, i], state)
            ys.append(y)
            if i in (P - 1, L - 1):
                tag = "mid" if i == P - 1 else "end"
                for layer, (S, z) in enumerate(state):
                    # copies: the reference updates the state tensors in place on the next step
                    blob["%s_S%d" % (tag, layer)] = np_(S.clone())
                    blob["%s_z%d" % (tag, layer)] = np_(z.clone())
    blob["y"] = np_(torch.stack(ys, 1))
    blob["prefix"] = np.int64(P)
    np.savez_compressed(os.path.join(HERE, "recurrent_encoder.npz"), **blob)
    print("recurrent_encoder.npz", os.path.getsize(os.path.join(HERE, "recurrent_encoder.npz")), "bytes")


def linear():
    """``linear.npz``: the reference's unmasked ``LinearAttention`` (inputs with keys longer than
    queries and ragged key lengths, output, gradients of a weighted sum) and its
    ``RecurrentCrossLinearAttention`` stepped over a few queries on the same memory (every output,
    the state), with the check that the steps reproduce the batch form."""
    import_reference_recurrent()
    pkg_dir = os.path.join(build_ref.reference_root(), "fast_transformers")
    m = types.ModuleType("fast_transformers.recurrent.attention.cross_attention")
    m.__path__ = [os.path.join(pkg_dir, "recurrent/attention/cross_attention")]
    sys.modules["fast_transformers.recurrent.attention.cross_attention"] = m
    import fast_transformers.attention.linear_attention as la
    import fast_transformers.recurrent.attention.cross_attention.linear_attention as rcla
    import fast_transformers.masking as masking
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(808)
    N, L, S, H, E, M = 3, 9, 14, 4, 16, 24
    q = torch.randn(N, L, H, E, generator=g, requires_grad=True)
    k = torch.randn(N, S, H, E, generator=g, requires_grad=True)
    v = torch.randn(N, S, H, M, generator=g, requires_grad=True)
    w = torch.randn(N, L, H, M, generator=g)
    klen = torch.tensor([14, 5, 11])
    att = la.LinearAttention(E).eval()
    qlm = masking.LengthMask(torch.full((N,), L, dtype=torch.long))
    klm = masking.LengthMask(klen, max_len=S)
    y = att(q, k, v, masking.FullMask(L, S), qlm, klm)
    (y * w).sum().backward()
    blob = {"q": np_(q), "k": np_(k), "v": np_(v), "w": np_(w), "klen": np_(klen), "y": np_(y),
            "gq": np_(q.grad), "gk": np_(k.grad), "gv": np_(v.grad)}
    rec = rcla.RecurrentCrossLinearAttention(E).eval()
    with torch.no_grad():
        state, ys = None, []
        for i in range(L):
            yi, state = rec(q[:, i], k, v, klm, state)
            ys.append(yi)
    blob["step_y"] = np_(torch.stack(ys, 1))
    blob["state_S"] = np_(state[0])      # (N, H, M, E) in the reference
    blob["state_z"] = np_(state[1])
    assert np.abs(blob["step_y"] - blob["y"]).max() < 1e-5
    np.savez_compressed(os.path.join(HERE, "linear.npz"), **blob)
    print("linear.npz", os.path.getsize(os.path.join(HERE, "linear.npz")), "bytes")


def favor_wide():
    """``favor64.npz``: the reference's ``Favor`` on 64-wide inputs with 256 features (the shape of
    configuration 5 and of the native feature-map kernel): omega, inputs, features, and the
    gradient of a weighted sum with respect to the inputs."""
    cp, cla, al, fm, masking, tr = import_reference()
    from fast_transformers_b200 import workloads
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(909)
    E, n_dims = 64, 256
    f = fm.Favor(E, n_dims=n_dims)
    omega = workloads.favor_omega(E, n_dims, g)
    f.omega.copy_(omega)
    x = (torch.randn(1, 19, 2, E, generator=g) * 0.5).requires_grad_(True)
    w = torch.rand(1, 19, 2, n_dims, generator=g)
    phi = f(x)
    (phi * w).sum().backward()
    np.savez_compressed(os.path.join(HERE, "favor64.npz"), omega=np_(omega), x=np_(x), w=np_(w),
                        phi=np_(phi), gx=np_(x.grad))
    print("favor64.npz", os.path.getsize(os.path.join(HERE, "favor64.npz")), "bytes")


def product_wide():
    """``product_wide.npz``: the reference's product and gradients for query / value widths that are
    multiples of 64 above 64 (every eighth row from row 3 on, plus checksums of the whole tensors);
    the inputs are ``fast_transformers_b200.workloads.wide_golden_inputs``."""
    cp, cla, al, fm, masking, tr = import_reference()
    from fast_transformers_b200 import workloads
    torch.set_num_threads(1)
    blob = {}
    for D, M in workloads.WIDE_GOLDEN_SHAPES:
        Q, K, V, G = workloads.wide_golden_inputs(D, M)
        Qr, Kr, Vr = (t.clone().requires_grad_(True) for t in (Q, K, V))
        out = cp.causal_dot_product(Qr, Kr, Vr)
        out.backward(G)
        for name, t in (("out", out), ("gQ", Qr.grad), ("gK", Kr.grad), ("gV", Vr.grad)):
            blob["%s_%d_%d" % (name, D, M)] = np_(t[:, :, workloads.WIDE_GOLDEN_ROWS])
            blob["sum_%s_%d_%d" % (name, D, M)] = np.array(t.double().sum().item())
    np.savez_compressed(os.path.join(HERE, "product_wide.npz"), **blob)
    print("product_wide.npz", os.path.getsize(os.path.join(HERE, "product_wide.npz")), "bytes")


if __name__ == "__main__":
    if sys.argv[1:] == ["favor_wide"]:
        favor_wide()
    elif sys.argv[1:] == ["product_wide"]:
        product_wide()
    elif sys.argv[1:] == ["linear"]:
        linear()
    elif sys.argv[1:] == ["recurrent"]:
        recurrent()
    elif sys.argv[1:] == ["recurrent_encoder"]:
        recurrent_encoder()
    else:
        main()
        recurrent()
        recurrent_encoder()
        linear()
        favor_wide()
        product_wide()
