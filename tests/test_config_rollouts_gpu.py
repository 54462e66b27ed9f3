"""The rollout configurations of the benchmark contract at their full sizes, on the GPU, against
the reference's own CUDA code compiled from its sources (oracle/_ref/, skipped where absent):

* full game, 262,144 envs, 3 MinGRU layers, seed 2, 256 rollout steps with auto-reset: the
  reference's CUDA env writes the 996-byte records on the device (k_record_obs), this library's
  fused forward drives the env with its sampled actions, the reference's strict-fp32 cuBLAS
  pipeline reads the same records and prev_terminals, every step compared on the device;
* classic game, 1,048,576 envs, 3 layers, seed 3, 128 steps with auto-reset: the same with the
  reference's classic env kernels and its record-driven classic pipeline.

Both sides keep their own recurrent state for the whole rollout (free-running), so operand
rounding accumulates as it would in `run`.  Acceptance bounds of the path: max |dlogit| and
|dvalue| <= 2e-2, greedy-action agreement >= 99.5 % of env-steps; the agreement of the SAMPLED
actions (same Philox draw on both sides) is printed beside them.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H = 256


def _report(tag, r):
    print(f"[{tag}] env-steps={r['env_steps']:.0f} max|dlogit|={r['max_dlogit']:.3e} "
          f"max|dvalue|={r['max_dvalue']:.3e} greedy={r['greedy_agreement']:.5f} "
          f"sampled={r['sampled_agreement']:.5f} episode_ends={r['episode_ends']:.0f} "
          f"max|logit|={r['max_logit']:.2f}")


@pytest.mark.parametrize("n,steps,layers", [(4096, 32, 2), (262144, 256, 3)],
                         ids=["4096x32-L2", "262144x256-L3"])
def test_full_game_rollout_against_reference_fp32_pipeline(cfx, gpu, oracle, n, steps, layers):
    if not oracle.RefCuda.available(layers):
        pytest.skip(f"oracle/_ref/libcfref_cuda_l{layers}.so not built (reference sources absent)")
    cfx.lib()
    params = oracle.init_weights(H, layers, 43, seed=2)          # N(0, 1/fan_in), zero biases
    try:
        r = oracle.RefCuda.lockstep(layers, n, steps, 2, params, cfx.PREC_F16)
    except RuntimeError as e:
        if "without the lock-step loop" in str(e):
            pytest.skip(str(e))
        raise
    _report(f"full game {n} envs x {steps} steps L={layers}, f16 vs reference fp32 cuBLAS", r)
    assert r["env_steps"] == n * steps
    assert r["max_dlogit"] <= 2e-2 and r["max_dvalue"] <= 2e-2
    assert r["greedy_agreement"] >= 0.995
    if steps >= 256:
        assert r["episode_ends"] > 0          # auto-reset was exercised


def test_full_game_rollout_single_step_gate(cfx, gpu, oracle):
    """The same loop with the reference's recurrent state re-synchronised from this library's
    before every step: the bounds then measure one forward, not drift."""
    if not oracle.RefCuda.available(3):
        pytest.skip("oracle/_ref/libcfref_cuda_l3.so not built (reference sources absent)")
    cfx.lib()
    params = oracle.init_weights(H, 3, 43, seed=2)
    try:
        r = oracle.RefCuda.lockstep(3, 65536, 64, 2, params, cfx.PREC_F16, sync_state=1)
    except RuntimeError as e:
        if "without the lock-step loop" in str(e):
            pytest.skip(str(e))
        raise
    _report("full game 65536 envs x 64 steps L=3, single-step, f16 vs reference fp32 cuBLAS", r)
    assert r["max_dlogit"] <= 2e-2 and r["max_dvalue"] <= 2e-2
    assert r["greedy_agreement"] >= 0.995


@pytest.mark.parametrize("n,steps", [(8192, 32), (1048576, 128)], ids=["8192x32", "1048576x128"])
def test_classic_rollout_against_reference_classic_pipeline(cfx, gpu, oracle, n, steps):
    if not oracle.RefClassic.available():
        pytest.skip("oracle/_ref/libcfref_classic.so not built (reference sources absent)")
    cfx.lib()
    ref = oracle.RefClassic()
    params = oracle.classic_init_weights(H, 3, 17, seed=3)
    try:
        r = ref.lockstep(n, steps, 3, params, cfx.PREC_F16, tf32=0)
    except RuntimeError as e:
        if "without the lock-step loop" in str(e):
            pytest.skip(str(e))
        raise
    _report(f"classic {n} envs x {steps} steps L=3, f16 vs reference classic kernels + fp32 cuBLAS", r)
    assert r["env_steps"] == n * steps
    assert r["max_dlogit"] <= 2e-2 and r["max_dvalue"] <= 2e-2
    assert r["greedy_agreement"] >= 0.995
    if steps >= 128:
        assert r["episode_ends"] > 0
