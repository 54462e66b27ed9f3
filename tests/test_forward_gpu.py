"""GPU parity tests of the forward through the C ABI against the CPU oracle."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, L, A = 256, 2, 43


def run_steps(cfx, oracle, pol, params, recs, terms, uniforms, state0=None, check_state=True):
    """Feeds T steps to the device policy and the oracle (free-running states);
    returns per-step (device dict, oracle logits, oracle actions, oracle logprobs)."""
    T, n = recs.shape[:2]
    st = np.zeros((pol.L, n, pol.H), np.float32) if state0 is None else state0.copy()
    pol.set_state(st)
    out = []
    for t in range(T):
        d = pol.forward_host(recs[t], terms[t], uniforms[t])
        d = {k: v.copy() for k, v in d.items()}
        lav = oracle.forward(params, recs[t], terms[t], st, pol.H, pol.L, pol.A)
        a, lp = oracle.sample(lav, uniforms[t], pol.A)
        out.append((d, lav, a, lp))
    return out, st


def test_expand_bit_exact(cfx, gpu, oracle, golden_env):
    rec = golden_env["records"].reshape(-1, 996)
    got = cfx.expand_obs(rec)
    want = oracle.expand(rec)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    rec2 = np.random.default_rng(0).integers(0, 256, (96, 996), dtype=np.uint8)
    assert np.array_equal(cfx.expand_obs(rec2).view(np.uint32), oracle.expand(rec2).view(np.uint32))


def test_sampler_matches_oracle(cfx, gpu, oracle):
    rng = np.random.default_rng(3)
    lg = rng.normal(0, 1.5, (8192, 44)).astype(np.float32)
    u = rng.random(8192, dtype=np.float32)
    u[:4] = [1.0, 1e-9, 0.5, 0.999999]
    a, lp = cfx.sample_actions(lg, u)
    wa, wlp = oracle.sample(lg, u)
    # expf/logf differ by an ulp between glibc and CUDA: allow a handful of CDF ties
    assert (a != wa).sum() <= 2
    same = a == wa
    assert np.abs(lp[same] - wlp[same]).max() < 2e-6


def test_philox_uniforms(cfx, gpu):
    u = cfx.philox_uniforms(42, 0, 7, 4096)
    assert u.min() > 0.0 and u.max() <= 1.0
    assert abs(u.mean() - 0.5) < 0.02
    again = cfx.philox_uniforms(42, 0, 7, 4096)
    assert np.array_equal(u, again)
    # the subsequence is the global env index: a shifted window reproduces the tail
    shifted = cfx.philox_uniforms(42, 1024, 7, 1024)
    assert np.array_equal(shifted, u[1024:2048])
    assert not np.array_equal(cfx.philox_uniforms(42, 0, 8, 4096), u)


def test_strict_forward_matches_oracle_on_env_records(cfx, gpu, oracle, golden_env, golden_oracle):
    recs, terms = golden_env["records"], golden_env["prev_terminals"]
    n = recs.shape[1]
    params = oracle.init_weights(H, L, A, seed=int(golden_oracle["weight_seed"]))
    pol = cfx.Policy(n, H, L, A, "fp32")
    pol.set_weights(params)
    assert np.array_equal(pol.get_weights(), params)
    out, st = run_steps(cfx, oracle, pol, params, recs, terms, golden_oracle["uniforms"])
    for t, (d, lav, a, lp) in enumerate(out):
        assert np.abs(d["logits_av"] - lav).max() < 2e-5, t
        assert np.abs(d["logits_av"] - golden_oracle["logits_av"][t]).max() < 2e-5
        assert np.array_equal(d["values"], d["logits_av"][:, A])
        assert (d["actions"] != a).sum() <= 1
        assert np.array_equal(d["env_actions"], d["actions"].astype(np.float32))
        same = d["actions"] == a
        assert np.abs(d["logprobs"][same] - lp[same]).max() < 1e-5
    assert np.abs(pol.get_state() - st).max() < 2e-5
    assert pol.last_launches == 1 + L + 2
    pol.close()


@pytest.mark.parametrize("n,layers,hidden,scheme", [(32, 2, 256, "uniform"), (96, 3, 256, "normal"),
                                                    (160, 2, 128, "uniform"), (64, 1, 512, "normal")])
def test_strict_forward_shapes(cfx, gpu, oracle, n, layers, hidden, scheme):
    rng = np.random.default_rng(n)
    rec = oracle.synthetic_records(n, seed=4)
    params = oracle.init_weights(hidden, layers, A, seed=5, scheme=scheme)
    state = rng.normal(0, 1, (layers, n, hidden)).astype(np.float32)
    prev_t = (rng.random(n) < 0.3).astype(np.float32)
    u = rng.random(n, dtype=np.float32)
    pol = cfx.Policy(n, hidden, layers, A, "fp32")
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, prev_t, u, want_r_state=True)
    st = state.copy()
    lav, rs = oracle.forward(params, rec, prev_t, st, hidden, layers, A, want_r_state=True)
    scale = max(1.0, np.abs(lav).max())
    assert np.abs(d["logits_av"] - lav).max() < 3e-5 * scale
    assert np.abs(pol.get_state() - st).max() < 3e-5 * max(1.0, np.abs(st).max())
    assert np.array_equal(d["r_state"], rs)
    pol.close()


def test_internal_philox_sampling_and_step_counter(cfx, gpu, oracle):
    n = 128
    rec = oracle.synthetic_records(n, seed=1)
    params = oracle.init_weights(H, L, A, seed=2)
    pol = cfx.Policy(n, H, L, A, "fp32")
    pol.set_weights(params)
    assert pol.step == 0
    d0 = {k: v.copy() for k, v in pol.forward_host(rec, None, None, seed=99, bump_step=True).items()}
    assert pol.step == 1
    u0 = cfx.philox_uniforms(99, 0, 0, n)
    a0, lp0 = cfx.sample_actions(d0["logits_av"], u0)
    assert np.array_equal(a0, d0["actions"]) and np.array_equal(lp0, d0["logprobs"])
    # replay: same step + same state gives identical outputs
    pol.step = 0
    pol.reset_state()
    d1 = pol.forward_host(rec, None, None, seed=99, bump_step=False)
    assert np.array_equal(d1["actions"], d0["actions"])
    assert np.array_equal(d1["logits_av"], d0["logits_av"])
    # env_offset shifts the Philox subsequence (contiguous-slice sharding)
    pol.step = 0
    pol.reset_state()
    d2 = pol.forward_host(rec, None, None, seed=99, env_offset=1000)
    u2 = cfx.philox_uniforms(99, 1000, 0, n)
    assert np.array_equal(cfx.sample_actions(d2["logits_av"], u2)[0], d2["actions"])
    pol.close()


def test_checkpoint_roundtrip_and_errors(cfx, gpu, oracle, tmp_path):
    pol = cfx.Policy(32, H, L, A, "fp32")
    pol.init_weights(1234)
    w = pol.get_weights()
    o = oracle.offsets(H, L, A)
    assert np.abs(w[:o["b_enc"]]).max() <= 1 / np.sqrt(843) and w.std() > 0
    assert np.abs(w[o["w_gru"]:o["w_a"]]).max() <= 1 / 16 + 1e-7
    path = str(tmp_path / "w.cfw1")
    pol.save(path)
    raw = np.fromfile(path, np.uint32, 4)
    assert list(raw) == [0x31574643, H, L, w.size]
    assert os.path.getsize(path) == 16 + 4 * w.size
    pol2 = cfx.Policy(32, H, L, A, "fp32")
    pol2.load(path)
    assert np.array_equal(pol2.get_weights(), w)
    pol3 = cfx.Policy(32, H, 3, A, "fp32")
    with pytest.raises(cfx.CfxError):
        pol3.load(path)            # layer count mismatch in the header
    with pytest.raises(cfx.CfxError):
        pol2.load(str(tmp_path / "missing"))
    with open(path, "r+b") as f:
        f.truncate(1000)
    with pytest.raises(cfx.CfxError):
        pol2.load(path)            # truncated
    with pytest.raises(cfx.CfxError):
        pol.set_weights(w[:-1])
    for p in (pol, pol2, pol3):
        p.close()
