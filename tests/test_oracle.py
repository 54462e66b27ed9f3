"""CPU tests of the oracle: against the committed fixtures, against an independent
float64 numpy statement of the same network, and of the record layout as produced
by the reference's own C environment."""
import numpy as np
import pytest

H, L, A = 256, 2, 43


def np_forward64(O, params, rec, prev_t, state):
    """Vectorised float64 forward; an independent statement of the same network
    (Linear 843->H, L MinGRU layers, actor+value heads)."""
    o = O.offsets(H, L, A)
    p = params.astype(np.float64)
    x = O.expand(rec).astype(np.float64)
    W_enc = p[o["w_enc"]:o["b_enc"]].reshape(O.OBS, H)
    h = x @ W_enc + p[o["b_enc"]:o["w_gru"]]
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    keep = (prev_t == 0)[:, None]
    new_state = np.empty_like(state, dtype=np.float64)
    for l in range(L):
        W = p[o["w_gru"] + l * 3 * H * H: o["w_gru"] + (l + 1) * 3 * H * H].reshape(3 * H, H)
        pre = h @ W.T
        zh, zg, zp = pre[:, :H], pre[:, H:2 * H], pre[:, 2 * H:]
        st = state[l].astype(np.float64) * keep
        g = np.where(zh >= 0, zh + 0.5, sig(zh))
        out = st + sig(zg) * (g - st)
        pp = sig(zp)
        h = pp * out + (1 - pp) * h
        new_state[l] = out
    logits = h @ p[o["w_a"]:o["b_a"]].reshape(A, H).T + p[o["b_a"]:o["w_v"]]
    value = h @ p[o["w_v"]:o["b_v"]] + p[o["b_v"]]
    return np.concatenate([logits, value[:, None]], 1), new_state


def test_param_count(oracle):
    assert oracle.param_count(256, 2, 43) == 620588   # CF_NN_PARAM_COUNT at h256x2
    assert oracle.param_count(256, 3, 43) == 817196
    assert oracle.offsets(256, 2, 43)["count"] == 620588


def test_expand_is_exact(oracle, golden_env):
    rec = golden_env["records"][0]
    x = oracle.expand(rec)
    assert x.dtype == np.float32 and x.shape == (rec.shape[0], 843)
    assert np.array_equal(x[:, :792], rec[:, :792].astype(np.float32))
    assert np.array_equal(x[:, 792:].view(np.uint32), rec[:, 792:].copy().view(np.uint32))


def test_expand_every_byte_value(oracle):
    rec = np.zeros((256, 996), np.uint8)
    rec[:, :792] = np.arange(256, dtype=np.uint8)[:, None]
    rec[:, 792:] = np.random.default_rng(0).integers(0, 256, (256, 204), dtype=np.uint8)
    x = oracle.expand(rec)
    assert np.array_equal(x[:, 0], np.arange(256, dtype=np.float32))
    assert np.array_equal(x[:, 792:].view(np.uint32), rec[:, 792:].copy().view(np.uint32))


def test_record_layout_from_reference_env(golden_env):
    """Layout facts of craftax_full.c:565-581 on records the reference env wrote."""
    rec = golden_env["records"]
    m = rec[..., :792].reshape(*rec.shape[:2], 99, 8)
    assert m[..., 0].max() <= 36 and m[..., 1].max() <= 5 and m[..., 2].max() <= 1
    assert m[..., 3:].max() <= 8
    invisible = m[..., 2] == 0
    assert np.all(m[invisible] == 0) or np.all(m[invisible][:, 3:] == 0)
    tail = rec[..., 792:].copy().view(np.float32)
    assert tail.shape[-1] == 51 and np.isfinite(tail).all()
    assert tail.min() >= 0.0 and tail.max() <= 1.0 + 1e-6
    assert np.all(tail[..., 31:35].sum(-1) == 1.0)  # direction one-hot


def test_forward_matches_golden(oracle, golden_env, golden_oracle):
    params = oracle.init_weights(H, L, A, seed=int(golden_oracle["weight_seed"]))
    n = golden_env["records"].shape[1]
    state = np.zeros((L, n, H), np.float32)
    for t in range(golden_env["records"].shape[0]):
        lav = oracle.forward(params, golden_env["records"][t], golden_env["prev_terminals"][t], state)
        assert np.array_equal(lav, golden_oracle["logits_av"][t]), t
        a, lp = oracle.sample(lav, golden_oracle["uniforms"][t])
        assert np.array_equal(a, golden_oracle["actions"][t])
        assert np.array_equal(lp, golden_oracle["logprobs"][t])
    assert np.array_equal(state, golden_oracle["final_state"])


def test_forward_matches_float64_statement(oracle, golden_env):
    params = oracle.init_weights(H, L, A, seed=3, scheme="uniform")
    rec = golden_env["records"][5]
    n = rec.shape[0]
    rng = np.random.default_rng(2)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.25).astype(np.float32)
    want, want_state = np_forward64(oracle, params, rec, prev_t, state)
    st = state.copy()
    got, h, rs = oracle.forward(params, rec, prev_t, st, want_h=True, want_r_state=True)
    assert np.abs(got - want).max() < 2e-5
    assert np.abs(st - want_state).max() < 2e-5
    assert np.array_equal(rs, state * (prev_t == 0)[None, :, None])
    assert h.shape == (n, H)


def test_thread_count_does_not_change_results(oracle, golden_env):
    params = oracle.init_weights(H, L, A, seed=1)
    rec = golden_env["records"][0]
    s1 = np.zeros((L, 64, H), np.float32)
    s2 = np.zeros((L, 64, H), np.float32)
    a = oracle.forward(params, rec, None, s1, threads=1)
    b = oracle.forward(params, rec, None, s2, threads=max(2, oracle.max_threads()))
    assert np.array_equal(a, b) and np.array_equal(s1, s2)


def test_sampler_semantics(oracle):
    rng = np.random.default_rng(5)
    lg = rng.normal(0, 2, (4096, 44)).astype(np.float32)
    u = rng.random(4096, dtype=np.float32)
    a, lp = oracle.sample(lg, u)
    p = np.exp(lg[:, :43].astype(np.float64) - lg[:, :43].max(1, keepdims=True))
    cdf = np.cumsum(p, 1) / p.sum(1, keepdims=True)
    want = np.minimum((cdf < u[:, None]).sum(1), 42)
    assert (a == want).mean() > 0.999          # float32 vs float64 CDF ties only
    lsm = lg[:, :43] - lg[:, :43].max(1, keepdims=True) - np.log(p.sum(1, keepdims=True))
    assert np.abs(lp - lsm[np.arange(4096), a]).max() < 1e-5
    # u = 1.0 (curand_uniform's upper end) with a huge last logit gap still returns a valid index
    a1, _ = oracle.sample(lg[:8], np.ones(8, np.float32))
    assert a1.min() >= 0 and a1.max() <= 42
    # empirical frequencies follow softmax
    one = np.tile(np.array([[0.0, 1.0, 2.0] + [-30.0] * 41], np.float32), (20000, 1))
    af, _ = oracle.sample(one, rng.random(20000, dtype=np.float32))
    freq = np.bincount(af, minlength=43)[:3] / 20000
    sm = np.exp([0.0, 1.0, 2.0]) / np.exp([0.0, 1.0, 2.0]).sum()
    assert np.abs(freq - sm).max() < 0.015


def test_state_zeroed_on_prev_terminal(oracle, golden_env):
    params = oracle.init_weights(H, L, A, seed=4)
    rec = golden_env["records"][1]
    rng = np.random.default_rng(9)
    state = rng.normal(0, 1, (L, 64, H)).astype(np.float32)
    zero = np.zeros_like(state)
    t = np.ones(64, np.float32)
    a = oracle.forward(params, rec, t, state.copy())
    b = oracle.forward(params, rec, None, zero.copy())
    assert np.array_equal(a, b)


@pytest.mark.skipif("not __import__('oracle').RefEnv.available()")
def test_reference_env_is_deterministic_and_matches_fixture(oracle, golden_env):
    env = oracle.RefEnv(int(golden_env["num_envs"]), int(golden_env["seed"]))
    for _ in range(int(golden_env["first_step"])):
        env.step_random()
    assert np.array_equal(env.records, golden_env["records"][0])
    assert np.array_equal(env.terminals, golden_env["prev_terminals"][0])
    env.close()
