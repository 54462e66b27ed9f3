"""Lock-step rollouts on the GPU: the fused kernel's sampled actions drive the reference's own
C environment (compact-obs build), and every step's logits are compared with an fp32 run of
the same policy on the same records. Both sides carry their OWN recurrent state for the whole
rollout, so operand-rounding error is allowed to accumulate the way it would in `run`.

Bounds (the acceptance bounds of the path): max |dlogit|, |dvalue| <= 2e-2 against the fp32
path, greedy-action agreement >= 99.5 %.  The fp32 side is the reference's cuBLAS pipeline in
strict-fp32 math mode where its library was built, else the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, A = 256, 43


class _Fp32Side:
    """fp32 run of the policy with its own recurrent state: reference pipeline or oracle."""

    def __init__(self, cfx, oracle, params, n, layers):
        self.cfx, self.oracle, self.params, self.n, self.layers = cfx, oracle, params, n, layers
        o = oracle.offsets(H, layers, A)
        self.bias = np.concatenate([params[o["b_a"]:o["w_v"]], params[o["b_v"]:o["b_v"] + 1]])
        self.ref = None
        if oracle.RefCuda.available(layers):
            self.ref = oracle.RefCuda(n, layers)
            self.ref.set_weights(params)
            self.ref.set_state(self.ref.FP32, np.zeros((layers, n, H), np.float32))
            self.kind = "reference fp32 cuBLAS pipeline"
        else:
            self.state = np.zeros((layers, n, H), np.float32)
            self.kind = "CPU oracle"

    def step(self, rec, prev_t):
        if self.ref is not None:
            d_rec = self.cfx.DeviceBuffer.from_host(rec)
            d_pt = self.cfx.DeviceBuffer.from_host(prev_t)
            r = self.ref.forward(self.ref.FP32, d_rec.ptr, d_pt.ptr, seed=1)
            return r["logits_nobias"] + self.bias[None, :]
        return self.oracle.forward(self.params, rec, prev_t, self.state, H, self.layers, A)

    def close(self):
        if self.ref is not None:
            self.ref.close()


def _lockstep(cfx, oracle, n, steps, layers, env_seed, weight_seed):
    env = oracle.RefEnv(n, env_seed)
    params = oracle.init_weights(H, layers, A, seed=weight_seed)
    pol = cfx.Policy(n, H, layers, A, "f16")
    pol.set_weights(params)
    side = _Fp32Side(cfx, oracle, params, n, layers)
    worst, agree, resets = 0.0, 0, 0
    hist = np.zeros(A, np.int64)
    for t in range(steps):
        rec, prev_t = env.records.copy(), env.terminals.copy()
        d = pol.forward_host(rec, prev_t, None, seed=99, bump_step=True)
        lav = side.step(rec, prev_t)
        worst = max(worst, float(np.abs(d["logits_av"] - lav).max()))
        agree += int((d["logits_av"][:, :A].argmax(1) == lav[:, :A].argmax(1)).sum())
        resets += int(prev_t.sum())
        hist += np.bincount(d["actions"], minlength=A)
        env.step(d["actions"].astype(np.float32))
    assert pol.step == steps             # the step counter is bumped inside the fused kernel
    # one launch per forward; from 65,536 envs the host-buffer entry point uploads the records in
    # slices of >= 32,768 envs and launches the kernel once per slice behind the copies
    assert pol.last_launches == max(1, min(8, n // 32768))
    pol.close(); side.close(); env.close()
    return worst, agree / (steps * n), resets, hist, side.kind


def test_lockstep_1024_envs_64_steps(cfx, gpu, oracle):
    if not oracle.RefEnv.available():
        pytest.skip("oracle/_ref/libcfref_env.so not built (reference sources absent)")
    worst, agree, resets, hist, kind = _lockstep(cfx, oracle, 1024, 64, 2, env_seed=0, weight_seed=42)
    print(f"[lock-step 1024x64 L=2 vs {kind}] max|dlogit|={worst:.3e} greedy={agree:.4f} "
          f"episode resets seen={resets}")
    assert worst <= 2e-2
    assert agree >= 0.995
    assert (hist > 0).sum() >= 40            # the sampler explores the action set


def test_lockstep_65536_envs_128_steps(cfx, gpu, oracle):
    """Full game at 65,536 envs for 128 rollout steps with auto-reset (seed 1): every step's
    logits and value against the reference's fp32 cuBLAS pipeline on the same records, both sides
    free-running."""
    if not oracle.RefEnv.available() or not oracle.RefCuda.available(2):
        pytest.skip("oracle/_ref libraries not built (reference sources absent)")
    worst, agree, resets, hist, kind = _lockstep(cfx, oracle, 65536, 128, 2, env_seed=1, weight_seed=43)
    print(f"[lock-step 65536x128 L=2 vs {kind}] max|dlogit|={worst:.3e} greedy={agree:.5f} "
          f"episode resets seen={resets}")
    assert worst <= 2e-2
    assert agree >= 0.995
    assert resets > 0


def test_lockstep_three_layers(cfx, gpu, oracle):
    if not oracle.RefEnv.available():
        pytest.skip("oracle/_ref/libcfref_env.so not built (reference sources absent)")
    worst, agree, _, _, kind = _lockstep(cfx, oracle, 512, 24, 3, env_seed=3, weight_seed=11)
    print(f"[lock-step 512x24 L=3 vs {kind}] max|dlogit|={worst:.3e} greedy={agree:.4f}")
    assert worst <= 2e-2
    assert agree >= 0.995


@pytest.mark.parametrize("prec", ["fp32", "f16"])
def test_env_slices_equal_the_whole_batch(cfx, gpu, oracle, prec):
    """Two ranks' contiguous env slices (env_offset = first env of the slice) reproduce the
    single-process result bit for bit: same logits, same Philox subsequences, same actions."""
    n, layers = 768, 2
    rng = np.random.default_rng(2)
    rec = oracle.synthetic_records(n, seed=31)
    params = oracle.init_weights(H, layers, A, seed=13)
    state = rng.normal(0, 1, (layers, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.1).astype(np.float32)

    def run(lo, hi):
        pol = cfx.Policy(hi - lo, H, layers, A, prec)
        pol.set_weights(params)
        pol.set_state(state[:, lo:hi])
        pol.step = 7
        d = pol.forward_host(rec[lo:hi], prev_t[lo:hi], None, seed=5, env_offset=lo)
        d = {k: v.copy() for k, v in d.items()}
        st = pol.get_state()
        pol.close()
        return d, st

    whole, st_w = run(0, n)
    parts = [run(0, 384), run(384, n)]
    for key in ("actions", "logprobs", "values", "logits_av"):
        got = np.concatenate([p[0][key] for p in parts])
        assert np.array_equal(got.view(np.uint32) if got.dtype == np.float32 else got,
                              whole[key].view(np.uint32) if got.dtype == np.float32 else whole[key]), key
    assert np.array_equal(np.concatenate([p[1] for p in parts], axis=1), st_w)
