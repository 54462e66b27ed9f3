"""Properties checked at the benchmark's full size (262,144 envs, h256x2) where the CPU oracle is
too slow: the fused kernel against the fp32 device path (itself pinned to the oracle and to the
reference's kernels at small sizes), invariance under env-slice sharding, determinism, and the
post-zero state record."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, L, A = 256, 2, 43
N = 262144


def _forward(cfx, prec, n, params, rec, prev_t, state, env_offset=0, want_r_state=False):
    pol = cfx.Policy(n, H, L, A, prec)
    pol.set_weights(params)
    pol.set_state(state)
    pol.step = 3
    d = pol.forward_host(rec, prev_t, None, seed=17, env_offset=env_offset, want_r_state=want_r_state)
    d = {k: v.copy() for k, v in d.items()}
    st = pol.get_state()
    pol.close()
    return d, st


def test_full_size_fused_forward_properties(cfx, gpu, oracle):
    rng = np.random.default_rng(2026)
    base = oracle.synthetic_records(8192, seed=4)
    rec = base[rng.integers(0, 8192, N)]
    params = oracle.init_weights(H, L, A, seed=0)
    state = rng.standard_normal((L, N, H), dtype=np.float32)
    prev_t = (rng.random(N) < 1.0 / 265.0).astype(np.float32)

    d16, st16 = _forward(cfx, "f16", N, params, rec, prev_t, state, want_r_state=True)
    d32, st32 = _forward(cfx, "fp32", N, params, rec, prev_t, state)

    # (1) against the fp32 path: synthetic records drive every channel over its full range, so
    # the bound is relative to the largest logit
    scale = max(4.0, float(np.abs(d32["logits_av"]).max()))
    err = float(np.abs(d16["logits_av"] - d32["logits_av"]).max())
    agree = float((d16["logits_av"][:, :A].argmax(1) == d32["logits_av"][:, :A].argmax(1)).mean())
    print(f"[262144 envs] max|dlogit|={err:.3e} (max|logit|={scale:.1f}) greedy={agree:.5f}")
    assert err < 5e-3 * scale
    assert agree >= 0.995
    assert np.abs(st16 - st32).max() < 5e-3 * max(4.0, float(np.abs(st32).max()))

    # (2) the state record is the previous state, zeroed where the episode ended
    want = state.copy()
    want[:, prev_t != 0] = 0
    assert np.array_equal(d16["r_state"], want)
    del want

    # (3) sampler outputs are consistent with the kernel's own logits for every env
    lav = d16["logits_av"]
    assert np.array_equal(d16["values"], lav[:, A])
    assert (d16["actions"] >= 0).all() and (d16["actions"] < A).all()
    m = lav[:, :A].max(1)
    lse = m + np.log(np.exp(lav[:, :A] - m[:, None]).sum(1))
    lp = lav[np.arange(N), d16["actions"]] - lse
    assert np.abs(lp - d16["logprobs"]).max() < 1e-4
    assert np.bincount(d16["actions"], minlength=A).min() > 0     # every action is drawn somewhere

    # (4) determinism, and invariance under sharding into env slices (what the ranks of a
    # multi-GPU run compute): same logits, actions, log-probs and state, bit for bit
    parts = []
    for lo, hi in ((0, N // 2), (N // 2, N)):
        parts.append(_forward(cfx, "f16", hi - lo, params, rec[lo:hi], prev_t[lo:hi], state[:, lo:hi],
                              env_offset=lo))
    for key in ("logits_av", "actions", "logprobs", "values"):
        got = np.concatenate([p[0][key] for p in parts])
        assert np.array_equal(got.view(np.uint32), d16[key].view(np.uint32)), key
    assert np.array_equal(np.concatenate([p[1] for p in parts], axis=1), st16)


def test_classic_large_batch_properties(cfx, gpu, oracle):
    """Classic game (148-byte records, 3 layers, 17 actions) at 262,144 envs: fused kernel against
    the fp32 device path, and env slices against the whole batch."""
    n, layers, actions = 262144, 3, 17
    rng = np.random.default_rng(7)
    base = oracle.classic_synthetic_records(8192, seed=15)
    rec = base[rng.integers(0, 8192, n)]
    params = oracle.classic_init_weights(H, layers, actions, seed=16)
    state = rng.standard_normal((layers, n, H), dtype=np.float32)
    flags = (rng.random(n) < 0.01).astype(np.float32)

    def run(prec, lo, hi):
        pol = cfx.Policy(hi - lo, H, layers, actions, prec, game="classic")
        pol.set_weights(params)
        pol.set_state(state[:, lo:hi])
        d = pol.forward_host(rec[lo:hi], flags[lo:hi], None, seed=5, env_offset=lo)
        d = {k: v.copy() for k, v in d.items()}
        st = pol.get_state()
        pol.close()
        return d, st

    d16, st16 = run("f16", 0, n)
    d32, st32 = run("fp32", 0, n)
    err = float(np.abs(d16["logits_av"] - d32["logits_av"]).max())
    agree = float((d16["logits_av"][:, :actions].argmax(1) == d32["logits_av"][:, :actions].argmax(1)).mean())
    print(f"[classic 262144 envs] max|dlogit|={err:.3e} greedy={agree:.5f}")
    assert err < 2e-2
    assert agree >= 0.995
    assert np.abs(st16 - st32).max() < 2e-2
    parts = [run("f16", 0, n // 2), run("f16", n // 2, n)]
    for key in ("logits_av", "actions", "logprobs", "values"):
        got = np.concatenate([p[0][key] for p in parts])
        assert np.array_equal(got.view(np.uint32), d16[key].view(np.uint32)), key
    assert np.array_equal(np.concatenate([p[1] for p in parts], axis=1), st16)
