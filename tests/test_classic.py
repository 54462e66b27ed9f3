"""Classic game (reference craftax_classic.cu): 148-byte record, 1345 one-hot / scalar features,
gather encoder, 3 MinGRU layers, 17 actions.  CPU tests pin the oracle's expand and encoder
against an independent numpy restatement of the feature layout; GPU tests compare the
library's fp32 path with the oracle through the C ABI."""
import numpy as np
import pytest

H, L, A = 256, 3, 17


def _numpy_expand(rec):
    """Feature layout written out independently of the C oracle (craftax_classic.cu:1265-1301)."""
    n = rec.shape[0]
    x = np.zeros((n, 1345), np.float32)
    blk = rec[:, :63].view(np.int8).astype(np.int64)
    mob = rec[:, 63:126].astype(np.int64)
    for cell in range(63):
        base = cell * 21
        ok = (blk[:, cell] >= 0) & (blk[:, cell] < 17)
        x[np.nonzero(ok)[0], base + blk[ok, cell]] = 1.0
        for j in range(4):
            x[:, base + 17 + j] = (mob[:, cell] >> j) & 1
    x[:, 1323:1339] = rec[:, 126:142].view(np.int8).astype(np.float32) / np.float32(10.0)
    d = rec[:, 142].view(np.int8)
    for k in range(4):
        x[:, 1339 + k] = d == k + 1
    x[:, 1343] = rec[:, 144:148].copy().view(np.float32).reshape(n)
    x[:, 1344] = rec[:, 143] != 0
    return x


def test_classic_oracle_expand_matches_numpy_layout(oracle):
    rec = oracle.classic_synthetic_records(257, seed=1)
    assert rec.shape == (257, 148)
    x = oracle.classic_expand(rec)
    assert np.array_equal(x, _numpy_expand(rec))
    assert 63 <= x[:, :1323].sum(1).min() and x[:, :1323].sum(1).max() <= 63 * 5


def test_classic_oracle_encoder_is_the_dense_product_of_its_expand(oracle):
    """The gather encoder adds exactly the W_enc rows the one-hot expand selects: a float64 dense
    product of expand(rec) with W_enc reproduces it to fp32 rounding."""
    n = 64
    rec = oracle.classic_synthetic_records(n, seed=2)
    params = oracle.classic_init_weights(H, L, A, seed=3)
    o = oracle.classic_offsets(H, L, A)
    assert params.size == o["count"] == 1345 * H + H + L * 3 * H * H + A * H + A + H + 1
    state = np.zeros((L, n, H), np.float32)
    lav, h_enc = oracle.classic_forward(params, rec, None, state, H, L, A, want_h_enc=True)
    W = params[:o["b_enc"]].reshape(1345, H).astype(np.float64)
    want = params[o["b_enc"]:o["w_gru"]].astype(np.float64) + _numpy_expand(rec).astype(np.float64) @ W
    assert np.abs(h_enc - want).max() < 5e-6
    assert lav.shape == (n, A + 1) and np.isfinite(lav).all()
    # done flags zero the recurrent state before the cell
    st1 = np.random.default_rng(0).normal(0, 1, (L, n, H)).astype(np.float32)
    st2 = st1.copy()
    done = np.zeros(n, np.int8); done[::2] = 1
    a = oracle.classic_forward(params, rec, done, st1, H, L, A)
    st2[:, ::2] = 0
    b = oracle.classic_forward(params, rec, None, st2, H, L, A)
    assert np.array_equal(a, b) and np.array_equal(st1, st2)


@pytest.mark.gpu
def test_classic_expand_kernel_is_bit_exact(cfx, gpu, oracle):
    rec = oracle.classic_synthetic_records(1000, seed=4)
    assert np.array_equal(cfx.classic_expand_obs(rec), oracle.classic_expand(rec))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [32, 1024 + 96])
def test_classic_forward_matches_oracle(cfx, gpu, oracle, n):
    rng = np.random.default_rng(n)
    rec = oracle.classic_synthetic_records(n, seed=5)
    params = oracle.classic_init_weights(H, L, A, seed=6)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    done = (rng.random(n) < 0.2).astype(np.int8)
    u = rng.random(n, dtype=np.float32)
    pol = cfx.Policy(n, H, L, A, "fp32", game="classic")
    assert pol.param_count == params.size
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, cfx.classic_done_to_terminals(done), u)
    want_st = state.copy()
    lav = oracle.classic_forward(params, rec, done, want_st, H, L, A)
    # same operation order on both sides; expf differs by an ulp between libm and CUDA
    assert np.abs(d["logits_av"] - lav).max() < 1e-5
    assert np.abs(pol.get_state() - want_st).max() < 1e-5
    a, lp = oracle.sample(lav, u, A)
    assert (a != d["actions"]).sum() <= 1
    assert np.array_equal(d["values"], d["logits_av"][:, A])
    # multi-step: state carried on both sides
    for t in range(3):
        rec_t = oracle.classic_synthetic_records(n, seed=10 + t)
        d = pol.forward_host(rec_t, None, None, seed=3, bump_step=True)
        lav = oracle.classic_forward(params, rec_t, None, want_st, H, L, A)
        assert np.abs(d["logits_av"] - lav).max() < 1e-4
    pol.close()


@pytest.mark.gpu
@pytest.mark.parametrize("prec,n", [("f16", 64), ("f16", 128 * 9 + 32), ("bf16", 256)])
def test_classic_fused_matches_oracle(cfx, gpu, oracle, prec, n):
    """Fused tcgen05 kernel on classic records: one-hot expand in tensor memory, dense encoder
    over the 1345 features, 3 layers, 17 actions; bounds as for the full game."""
    rng = np.random.default_rng(n)
    rec = oracle.classic_synthetic_records(n, seed=15)
    params = oracle.classic_init_weights(H, L, A, seed=16)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    done = (rng.random(n) < 0.2).astype(np.int8)
    u = rng.random(n, dtype=np.float32)
    pol = cfx.Policy(n, H, L, A, prec, game="classic")
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, done.astype(np.float32), u)
    assert pol.last_launches == 1
    want_st = state.copy()
    lav = oracle.classic_forward(params, rec, done, want_st, H, L, A)
    tol = 2e-2 if prec == "f16" else 1e-1
    err = float(np.abs(d["logits_av"] - lav).max())
    agree = float((d["logits_av"][:, :A].argmax(1) == lav[:, :A].argmax(1)).mean())
    print(f"[classic {prec} n={n}] max|dlogit|={err:.3e} greedy agreement={agree:.4f}")
    assert err < tol
    assert np.abs(pol.get_state() - want_st).max() < tol
    if prec == "f16":
        assert agree >= 0.995
    a, lp = cfx.sample_actions(d["logits_av"], u, num_actions=A)
    assert np.array_equal(a, d["actions"])
    assert np.array_equal(lp.view(np.uint32), d["logprobs"].view(np.uint32))
    assert np.array_equal(d["values"], d["logits_av"][:, A])
    pol.close()


@pytest.mark.gpu
def test_classic_fused_expand_is_exact(cfx, gpu, oracle):
    """Selection weights route features to the hidden units through exactly representable steps
    (zero gate weights: per layer h <- 0.125 + 0.5 h), so the in-kernel one-hot expand is checked
    bit for bit for every one of the 1323 one-hot features and the two flags."""
    n = 128
    rec = oracle.classic_synthetic_records(n, seed=17)
    x = oracle.classic_expand(rec)
    o = oracle.classic_offsets(H, L, A)
    pol = cfx.Policy(n, H, L, A, "f16", game="classic")
    exact = np.ones(1345, bool); exact[1323:1339] = False; exact[1343] = False   # counts / 10 and light round to fp16
    for base in range(0, 1345, H):
        for u0 in range(0, H, A):
            units = np.arange(u0, min(u0 + A, H))
            feats = base + units
            feats = feats[feats < 1345]
            units = units[:feats.size]
            if feats.size == 0:
                continue
            params = np.zeros(o["count"], np.float32)
            params[:o["b_enc"]].reshape(1345, H)[feats, units] = 1.0
            params[o["w_a"]:o["b_a"]].reshape(A, H)[np.arange(units.size), units] = 1.0
            pol.set_weights(params)
            pol.reset_state()
            d = pol.forward_host(rec, None, np.full(n, 0.5, np.float32))
            got = d["logits_av"][:, :units.size]
            want = 0.21875 + 0.125 * x[:, feats].astype(np.float64)     # three layers: 0.125 (1 + 0.5 + 0.25) + x / 8
            ex = exact[feats]
            assert np.array_equal(got[:, ex], want[:, ex].astype(np.float32)), (base, u0)
            if (~ex).any():
                assert np.abs(got[:, ~ex] - want[:, ~ex]).max() < 1e-3
    pol.close()


@pytest.mark.gpu
def test_classic_fused_modes_agree(cfx, gpu, oracle, monkeypatch):
    n = 128 * 5
    rng = np.random.default_rng(3)
    rec = oracle.classic_synthetic_records(n, seed=18)
    params = oracle.classic_init_weights(H, L, A, seed=19)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    out = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("CFX_FUSED_PAIR", mode)
        pol = cfx.Policy(n, H, L, A, "f16", game="classic")
        pol.set_weights(params)
        pol.set_state(state)
        d = pol.forward_host(rec, None, None, seed=4)
        out[mode] = ({k: v.copy() for k, v in d.items()}, pol.get_state())
        pol.close()
    assert np.array_equal(out["1"][0]["logits_av"], out["0"][0]["logits_av"])
    assert np.array_equal(out["1"][1], out["0"][1])
    assert np.array_equal(out["1"][0]["actions"], out["0"][0]["actions"])


@pytest.mark.gpu
def test_classic_against_the_reference_kernels(cfx, gpu, oracle):
    """Pins the classic oracle and the library against the REFERENCE's own kernels run on the
    same GPU: expand bit for bit, gather encoder and the whole forward to fp32 rounding (the
    reference's classic build uses --use_fast_math, so its sigmoid differs in the last bits),
    sampler bit-identical given the reference's logits and the same Philox draw."""
    if not oracle.RefClassic.available():
        pytest.skip("oracle/_ref/libcfref_classic.so not built (reference sources absent)")
    ref = oracle.RefClassic()
    assert (ref.H, ref.layers, ref.A) == (H, L, A)
    n = 512
    rng = np.random.default_rng(7)
    rec = oracle.classic_synthetic_records(n, seed=8)
    params = oracle.classic_init_weights(H, L, A, seed=9)
    assert params.size == ref.param_count
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    done = (rng.random(n) < 0.25).astype(np.int8)
    d_rec = cfx.DeviceBuffer.from_host(rec)
    d_par = cfx.DeviceBuffer.from_host(params)
    d_done = cfx.DeviceBuffer.from_host(done)
    d_state = cfx.DeviceBuffer.from_host(state)
    d_x = cfx.DeviceBuffer((n, 1345), np.float32)
    ref.expand(d_rec.ptr, d_x.ptr, n)
    x_ref = d_x.download()
    # one-hot features and the raw light level bit for bit; the 16 counts are divided by 10 with
    # the reference build's fast-math division, which may differ from IEEE division in the last bit
    x_or = oracle.classic_expand(rec)
    scaled = np.zeros(1345, bool); scaled[1323:1339] = True
    assert np.array_equal(x_ref[:, ~scaled], x_or[:, ~scaled])
    assert np.abs(x_ref[:, scaled] - x_or[:, scaled]).max() <= 6e-8
    assert np.array_equal(x_or, cfx.classic_expand_obs(rec))
    r = ref.forward(d_par.ptr, d_rec.ptr, d_done.ptr, d_state.ptr, n, seed=21, step=4)
    st_ref = d_state.download()
    st = state.copy()
    lav, h_enc = oracle.classic_forward(params, rec, done, st, H, L, A, want_h_enc=True)
    assert np.abs(r["h_enc"] - h_enc).max() < 2e-6               # same fmaf chain, same order
    assert np.abs(r["logits_av"] - lav).max() < 2e-4
    assert np.abs(st_ref - st).max() < 2e-4
    pol = cfx.Policy(n, H, L, A, "fp32", game="classic")
    pol.set_weights(params)
    pol.set_state(state)
    pol.step = 4
    d = pol.forward_host(rec, cfx.classic_done_to_terminals(done), None, seed=21)
    assert np.abs(d["logits_av"] - r["logits_av"]).max() < 2e-4
    assert np.abs(pol.get_state() - st_ref).max() < 2e-4
    assert (d["actions"] != r["actions"]).mean() < 0.01
    # sampler stage on the reference's logits with the reference's Philox stream
    u = cfx.philox_uniforms(21, 0, 4, n)
    a, lp = cfx.sample_actions(r["logits_av"], u, num_actions=A)
    assert np.array_equal(a, r["actions"])
    assert np.abs(lp - r["logprobs"]).max() < 1e-5             # its logf/expf are the fast-math ones
    pol.close()


@pytest.mark.gpu
@pytest.mark.parametrize("n,steps", [(4096 + 32, 160), (1048576, 3)], ids=["play-with-resets", "full-size"])
def test_classic_record_write_equals_the_reference_kernel(cfx, gpu, oracle, n, steps):
    """cfx_classic_record_obs writes the bytes record_obs_kernel writes (craftax_classic.cu:1574-1604,
    :1884-1890) from the reference's own classic device state, over random play with auto-reset."""
    if not oracle.RefClassic.available():
        pytest.skip("oracle/_ref/libcfref_classic.so not built (reference sources absent)")
    cfx.lib()
    r = oracle.RefClassic().record_parity(n, steps, seed=5)
    print(f"[classic record] n={n}: {r['rows_compared']:.0f} rows, {r['differing_bytes']:.0f} differing bytes, "
          f"{r['episode_ends']:.0f} episode ends; record_obs_kernel {r['reference_ms']:.4f} ms, "
          f"cfx_classic_record_obs {r['cfx_ms']:.4f} ms; {r['rows_with_mob']:.0f} of the last {n} rows show a mob")
    assert r["rows_compared"] == n * steps and r["differing_bytes"] == 0
    if steps > 100:
        assert r["rows_with_mob"] > 0 and r["episode_ends"] > 0
