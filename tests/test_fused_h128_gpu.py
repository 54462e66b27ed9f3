"""GPU parity tests of the hidden-128 instantiation of the fused kernel (the H = 128 points of the
sweep: two gate slices, two K blocks, four state boxes per layer, encoder N = 128), through the
C ABI against the CPU oracle and the fp32 device path."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
A = 43


def _run(cfx, n, hidden, layers, prec, params, rec, prev_t, u, state, **kw):
    pol = cfx.Policy(n, hidden, layers, A, prec)
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, prev_t, u, **kw)
    d = {k: v.copy() for k, v in d.items()}
    st = pol.get_state()
    launches = pol.last_launches
    pol.close()
    return d, st, launches


def _inputs(oracle, n, hidden, layers, seed, scheme="normal"):
    rng = np.random.default_rng(seed)
    base = oracle.synthetic_records(min(n, 4096), seed=seed + 1)
    rec = base if n <= 4096 else base[rng.integers(0, 4096, n)]
    params = oracle.init_weights(hidden, layers, A, seed=seed + 2, scheme=scheme)
    state = rng.normal(0, 1, (layers, n, hidden)).astype(np.float32)
    prev_t = (rng.random(n) < 0.2).astype(np.float32)
    u = rng.random(n, dtype=np.float32)
    return rec, params, state, prev_t, u


@pytest.mark.parametrize("prec,tol", [("f16", 2e-2), ("bf16", 1e-1)])
@pytest.mark.parametrize("n,layers", [(32, 2), (160, 3), (128 * 5 + 64, 2), (128 * 9, 1)])
def test_h128_fused_matches_oracle(cfx, gpu, oracle, n, layers, prec, tol):
    H = 128
    rec, params, state, prev_t, u = _inputs(oracle, n, H, layers, seed=n + layers, scheme="uniform")
    d, st, launches = _run(cfx, n, H, layers, prec, params, rec, prev_t, u, state)
    assert launches == 1
    want_st = state.copy()
    lav = oracle.forward(params, rec, prev_t, want_st, H, layers, A)
    assert np.abs(d["logits_av"] - lav).max() < tol
    assert np.abs(st - want_st).max() < tol
    a, lp = cfx.sample_actions(d["logits_av"], u)          # sampler on the kernel's own logits
    assert np.array_equal(a, d["actions"])
    assert np.array_equal(lp.view(np.uint32), d["logprobs"].view(np.uint32))
    assert np.array_equal(d["values"], d["logits_av"][:, A])


def test_h128_many_tiles_matches_strict_path(cfx, gpu, oracle):
    """More tiles than SMs (persistent loop, every ring wrapping) against the fp32 device path."""
    H, L = 128, 2
    n = 148 * 128 * 2 + 5 * 128 + 32
    rec, params, state, prev_t, _ = _inputs(oracle, n, H, L, seed=21)
    d0, st0, _ = _run(cfx, n, H, L, "fp32", params, rec, prev_t, None, state, seed=5)
    d1, st1, launches = _run(cfx, n, H, L, "f16", params, rec, prev_t, None, state, seed=5)
    assert launches == 1
    err = np.abs(d1["logits_av"] - d0["logits_av"]).max(1)
    scale = float(np.abs(d0["logits_av"]).max())
    print(f"h128 many tiles: max|dlogit|={err.max():.3e} max|logit|={scale:.2f}")
    assert err.max() < 5e-3 * max(scale, 4.0), (err.max(), int(err.argmax()))
    assert np.abs(st1 - st0).max() < 5e-3 * max(float(np.abs(st0).max()), 4.0)
    assert (d1["logits_av"][:, :A].argmax(1) == d0["logits_av"][:, :A].argmax(1)).mean() >= 0.995
    d2, st2, _ = _run(cfx, n, H, L, "f16", params, rec, prev_t, None, state, seed=5)
    assert np.array_equal(d1["logits_av"], d2["logits_av"]) and np.array_equal(st1, st2)


@pytest.mark.parametrize("n,layers", [(64, 2), (128 * 7, 3), (128 * 300 + 96, 2)])
def test_h128_single_cta_mode_equals_pair_mode(cfx, gpu, oracle, monkeypatch, n, layers):
    H = 128
    rec, params, state, prev_t, _ = _inputs(oracle, n, H, layers, seed=n)
    out = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("CFX_FUSED_PAIR", mode)
        out[mode] = _run(cfx, n, H, layers, "f16", params, rec, prev_t, None, state, seed=11,
                         want_r_state=True)
    (d1, st1, _), (d0, st0, _) = out["1"], out["0"]
    for key in ("logits_av", "actions", "logprobs", "r_state"):
        assert np.array_equal(d1[key], d0[key]), key
    assert np.array_equal(st1, st0)
    want = state.copy()
    want[:, prev_t != 0] = 0
    assert np.array_equal(d1["r_state"], want)


def test_h128_expand_is_exact_for_every_map_feature(cfx, gpu, oracle):
    """Selection weights route single features to the logits through exactly representable
    steps (zero gate weights: per layer h <- 0.125 + 0.5 h): every map byte bit for bit."""
    H, L, n = 128, 2, 128
    rng = np.random.default_rng(3)
    rec = oracle.synthetic_records(n, seed=12)
    rec[:, :792] = rng.integers(0, 256, (n, 792), dtype=np.uint8)
    x = oracle.expand(rec)
    o = oracle.offsets(H, L, A)
    pol = cfx.Policy(n, H, L, A, "f16")
    for base in list(range(0, 843 - H, H)) + [843 - H]:
        for u0 in range(0, H, A):
            units = np.arange(u0, min(u0 + A, H))
            params = np.zeros(o["count"], np.float32)
            params[:o["b_enc"]].reshape(843, H)[base + np.arange(H), np.arange(H)] = 1.0
            params[o["w_a"]:o["b_a"]].reshape(A, H)[np.arange(units.size), units] = 1.0
            pol.set_weights(params)
            pol.reset_state()
            d = pol.forward_host(rec, None, np.full(n, 0.5, np.float32))
            feats = base + units
            got = d["logits_av"][:, :units.size]
            want = 0.1875 + 0.25 * x[:, feats].astype(np.float64)
            is_map = feats < 792
            assert np.array_equal(got[:, is_map], want[:, is_map].astype(np.float32)), (base, u0)
            if (~is_map).any():
                assert np.abs(got[:, ~is_map] - want[:, ~is_map]).max() < 1e-3
    pol.close()


def test_hidden_512_has_no_fused_kernel(cfx, gpu, oracle):
    with pytest.raises(cfx.CfxError):
        cfx.Policy(64, 512, 2, A, "f16")
