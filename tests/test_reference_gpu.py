"""Pins the CPU oracle (and the strict CUDA path) against the REFERENCE's own CUDA code
run on the same GPU: its scalar fp32 policy kernel and its batched cuBLAS pipeline in
strict-fp32 math mode, compiled from the reference sources into oracle/_ref/ (prebuilt
where the sources live; skipped when that library was not built)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
H, L, A = 256, 2, 43


@pytest.fixture(scope="module")
def refcu(oracle, gpu):
    if not oracle.RefCuda.available(L):
        pytest.skip("oracle/_ref/libcfref_cuda_l2.so not built (reference sources absent)")
    return oracle.RefCuda


def _inputs(cfx, oracle, golden_env, n_rep=1, L=L):
    recs = golden_env["records"]
    rec = np.concatenate([recs[3]] * n_rep)
    n = rec.shape[0]
    rng = np.random.default_rng(21)
    state = rng.normal(0, 1, (L, n, H)).astype(np.float32)
    prev_t = (rng.random(n) < 0.2).astype(np.float32)
    return rec, state, prev_t, n


@pytest.mark.parametrize("scheme,L", [("normal", 2), ("uniform", 2), ("normal", 3)])
def test_oracle_matches_reference_scalar_kernel(cfx, oracle, refcu, golden_env, scheme, L):
    if not refcu.available(L):
        pytest.skip(f"oracle/_ref/libcfref_cuda_l{L}.so not built")
    rec, state, prev_t, n = _inputs(cfx, oracle, golden_env, L=L)
    params = oracle.init_weights(H, L, A, seed=7, scheme=scheme)
    ref = refcu(n, L)
    ref.set_weights(params)
    ref.set_step(5)
    ref.scalar_set_state(state)
    d_rec = cfx.DeviceBuffer.from_host(rec)
    d_pt = cfx.DeviceBuffer.from_host(prev_t)
    r = ref.scalar_forward(d_rec.ptr, d_pt.ptr, seed=17)
    st = state.copy()
    lav, h3 = oracle.forward(params, rec, prev_t, st, H, L, A, want_h=True)
    # same operation order on both sides; expf differs by an ulp between libm and CUDA
    assert np.abs(r["h3"] - h3).max() < 1e-5
    assert np.abs(r["values"] - lav[:, A]).max() < 1e-5
    assert np.abs(ref.scalar_get_state() - st).max() < 1e-5
    u = cfx.philox_uniforms(17, 0, 5, n)
    a, lp = oracle.sample(lav, u, A)
    assert (a != r["actions"]).sum() <= 1
    same = a == r["actions"]
    assert np.abs(lp[same] - r["logprobs"][same]).max() < 1e-5
    ref.close()


@pytest.mark.parametrize("L", [2, 3])
def test_strict_path_matches_reference_fp32_pipeline(cfx, oracle, refcu, golden_env, L):
    if not refcu.available(L):
        pytest.skip(f"oracle/_ref/libcfref_cuda_l{L}.so not built")
    rec, state, prev_t, n = _inputs(cfx, oracle, golden_env, n_rep=2, L=L)
    params = oracle.init_weights(H, L, A, seed=9)
    ref = refcu(n, L)
    ref.set_weights(params)
    ref.set_step(0)
    ref.set_state(ref.FP32, state)
    d_rec = cfx.DeviceBuffer.from_host(rec)
    d_pt = cfx.DeviceBuffer.from_host(prev_t)
    r = ref.forward(ref.FP32, d_rec.ptr, d_pt.ptr, seed=3)
    o = oracle.offsets(H, L, A)
    bias = np.concatenate([params[o["b_a"]:o["w_v"]], params[o["b_v"]:o["b_v"] + 1]])
    ref_lav = r["logits_nobias"] + bias[None, :]
    pol = cfx.Policy(n, H, L, A, "fp32")
    pol.set_weights(params)
    pol.set_state(state)
    d = pol.forward_host(rec, prev_t, None, seed=3)
    assert np.abs(d["logits_av"] - ref_lav).max() < 1e-4
    assert np.abs(pol.get_state() - ref.get_state(ref.FP32)).max() < 1e-4
    assert (d["actions"] != r["actions"]).mean() < 0.01
    # sampler stage: identical logits + identical uniforms -> identical bits
    u = cfx.philox_uniforms(3, 0, 0, n)
    a, lp = cfx.sample_actions(ref_lav, u)
    assert np.array_equal(a, r["actions"])
    assert np.array_equal(lp.view(np.uint32), r["logprobs"].view(np.uint32))
    assert np.array_equal(ref_lav[:, A].view(np.uint32), r["values"].view(np.uint32))
    pol.close()
    ref.close()


def test_expand_matches_reference_kernel_through_its_pipeline(cfx, oracle, refcu):
    """With W_enc a 0/1 selection matrix, zero biases and zero gate weights, the reference's
    strict-fp32 pipeline maps feature x to h3 through exactly representable steps
    (per layer: out = 0.25, p = 0.5, h = 0.5*0.25 + 0.5*h), so its k_expand_obs output is
    checked bit for bit through its own GEMM, and our expand against it."""
    n = 64
    rec = oracle.synthetic_records(n, seed=12)
    o = oracle.offsets(H, L, A)
    ours = cfx.expand_obs(rec)
    half, quarter = np.float32(0.5), np.float32(0.25)
    for base in (0, 256, 512, 843 - 256):
        params = np.zeros(o["count"], np.float32)
        W = params[:o["b_enc"]].reshape(843, H)
        W[base + np.arange(H), np.arange(H)] = 1.0
        ref = refcu(n, L)
        ref.set_weights(params)
        d_rec = cfx.DeviceBuffer.from_host(rec)
        r = ref.forward(ref.FP32, d_rec.ptr, None, seed=1)
        h = ours[:, base:base + H]
        for _ in range(L):
            h = half * quarter + half * h
        assert np.array_equal(r["h3"].view(np.uint32), h.astype(np.float32).view(np.uint32)), base
        ref.close()


def test_reference_run_loop_with_the_forward_swapped_in(cfx, oracle, refcu):
    """The reference's `run` loop (its env kernels, CUDA-graph replay) with the policy half
    replaced by cfx_policy_forward: the binding must capture into a graph, replay and leave no
    error behind; the unmodified loop runs beside it."""
    import ctypes as C
    if not refcu.available(2):
        pytest.skip("oracle/_ref/libcfref_cuda_l2.so not built")
    cfx.lib()
    lib = C.CDLL(refcu.path(2))
    if not hasattr(lib, "refcu_rollout_swap_sps"):
        pytest.skip("reference shim built without the swapped loop")
    lib.refcu_rollout_sps.restype = C.c_double
    lib.refcu_rollout_sps.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int]
    lib.refcu_rollout_swap_sps.restype = C.c_double
    lib.refcu_rollout_swap_sps.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int, C.c_int]
    ref_sps = lib.refcu_rollout_sps(4096, 40, 3, 1)
    for prec in (cfx.PREC_F16, cfx.PREC_FP32):
        sps = lib.refcu_rollout_swap_sps(4096, 40, 3, 1, prec)
        assert np.isfinite(sps) and sps > 0
        print(f"rollout 4096 envs: reference {ref_sps / 1e6:.1f} M SPS, swapped (precision {prec}) {sps / 1e6:.1f} M SPS")
    assert ref_sps > 0


@pytest.mark.parametrize("L", [2, 3])
def test_init_weights_equals_the_reference_initialiser(cfx, oracle, refcu, L):
    """cfx_policy_init_weights(1234) against the arena cu_policy_init writes
    (craftax_full.cu:11830-11845: Philox U(+-1/sqrt(fan_in)), seed 1234, one subsequence per
    segment), bit for bit."""
    if not refcu.available(L):
        pytest.skip(f"oracle/_ref/libcfref_cuda_l{L}.so not built")
    ref = refcu(32, L)
    want = ref.get_weights()          # untouched since cu_policy_init
    ref.close()
    pol = cfx.Policy(32, H, L, A, "fp32")
    pol.init_weights(1234)
    got = pol.get_weights()
    pol.close()
    assert got.size == want.size == cfx.lib().cfx_param_count(H, L, A)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.abs(want).max() > 0


@pytest.mark.parametrize("L", [2, 3])
def test_cfw1_files_cross_load_with_the_reference(cfx, oracle, refcu, L, tmp_path):
    """CFW1 checkpoints in both directions: a file written by the reference's cu_save_weights
    (craftax_full.cu:12248-12263) loads with cfx_policy_load_cfw1, and a file written by
    cfx_policy_save_cfw1 loads with cu_load_weights (:12264-12293); arenas and file bytes equal."""
    if not refcu.available(L):
        pytest.skip(f"oracle/_ref/libcfref_cuda_l{L}.so not built")
    ref = refcu(32, L)
    if not hasattr(ref.L, "refcu_save_cfw1"):
        pytest.skip("reference shim built without the checkpoint wrappers")
    params = oracle.init_weights(H, L, A, seed=31, scheme="uniform")
    # reference -> library
    ref.set_weights(params)
    f_ref = str(tmp_path / "from_reference.cfw1")
    ref.save_cfw1(f_ref)
    pol = cfx.Policy(32, H, L, A, "fp32")
    pol.load(f_ref)
    assert np.array_equal(pol.get_weights().view(np.uint32), params.view(np.uint32))
    # library -> reference
    params2 = oracle.init_weights(H, L, A, seed=32)
    pol.set_weights(params2)
    f_cfx = str(tmp_path / "from_library.cfw1")
    pol.save(f_cfx)
    assert ref.load_cfw1(f_cfx) == 0
    assert np.array_equal(ref.get_weights().view(np.uint32), params2.view(np.uint32))
    # same bytes for the same arena, whoever writes
    ref.save_cfw1(f_ref)
    assert open(f_ref, "rb").read() == open(f_cfx, "rb").read()
    # a file of another depth is refused by both sides
    other = cfx.Policy(32, H, 5 - L, A, "fp32")
    with pytest.raises(cfx.CfxError):
        other.load(f_cfx)
    other.close()
    pol.close()
    ref.close()


def test_play_recording_with_the_forward_swapped_in(cfx, oracle, refcu, tmp_path):
    """The reference's `play` mode (cu_run_play, craftax_full.cu:12383-12447: replay a policy from
    a CFW1 file, write one level/done byte per env and step and the CfFrame records of the
    chosen envs) with the policy half of every step taken from cfx_policy_forward: same
    recorders, same file formats; two runs with the same seed write identical files (what its
    --record-env workflow relies on), and the first step's actions agree with the reference's
    own play run on all but a few envs (fp16 against its default GEMM mode, same Philox draws)."""
    if not refcu.available(2):
        pytest.skip("oracle/_ref/libcfref_cuda_l2.so not built")
    cfx.lib()
    n, steps, recn, every = 1024, 12, 256, 4
    pol = cfx.Policy(32, H, L, A, "fp32")
    pol.init_weights(1234)
    wfile = str(tmp_path / "w.cfw1")
    pol.save(wfile)
    pol.close()
    out = {}
    try:
        for tag, swapped in (("ref", 0), ("cfx1", 1), ("cfx2", 1)):
            fr, lv = str(tmp_path / f"{tag}.frames"), str(tmp_path / f"{tag}.levels")
            fb, aoff = refcu.play(L, n, steps, 7, wfile, swapped, cfx.PREC_F16, recn, every, fr, lv)
            out[tag] = (open(fr, "rb").read(), open(lv, "rb").read())
    except RuntimeError as e:
        if "without the play loop" in str(e):
            pytest.skip(str(e))
        raise
    n_rec = (steps + every - 1) // every
    for tag in out:
        assert len(out[tag][1]) == n * steps, tag
        assert len(out[tag][0]) == n_rec * recn * fb, tag
    assert out["cfx1"] == out["cfx2"]                       # deterministic replay
    def actions(blob, k):
        fr = np.frombuffer(blob, np.uint8).reshape(n_rec, recn, fb)[k]
        return fr[:, aoff:aoff + 4].copy().view(np.int32)[:, 0]
    a_ref, a_cfx = actions(out["ref"][0], 0), actions(out["cfx1"][0], 0)
    assert (a_cfx >= 0).all() and (a_cfx < A).all()
    agree = float((a_ref == a_cfx).mean())
    print(f"[play] first-step action agreement with the reference's own play run: {agree:.4f}")
    assert agree >= 0.95


@pytest.mark.parametrize("n,steps,fuzz", [(2048, 96, 6), (262144, 4, 2)], ids=["play-and-fuzz", "full-size"])
def test_record_write_equals_the_reference_kernel(cfx, oracle, refcu, n, steps, fuzz):
    """cfx_record_obs writes the bytes k_record_obs writes (craftax_full.cu:9180-9297) from the
    reference's own device state: over random play with resets, on the just-reset envs through
    the list variant (k_record_obs_list), and on randomised state (mobs of every class on, off and
    at the edge of the view, type ids out of range, every level, unlit cells)."""
    if not refcu.available(2):
        pytest.skip("oracle/_ref/libcfref_cuda_l2.so not built")
    cfx.lib()
    r = refcu.record_parity(2, n, steps, fuzz, seed=11)
    print(f"[record] n={n}: {r['rows_compared']:.0f} rows, {r['differing_bytes']:.0f} differing bytes; "
          f"k_record_obs {r['reference_ms']:.4f} ms, cfx_record_obs {r['cfx_ms']:.4f} ms; "
          f"{r['rows_with_mob']:.0f} of the last {n} rows show a mob")
    assert r["rows_compared"] == n * (steps + fuzz)
    assert r["differing_bytes"] == 0
    assert r["list_differing_bytes"] == 0
    assert r["skip_differing_bytes"] == 0   # flagged envs are left untouched by both
    assert r["rows_with_mob"] > n // 4   # the randomised rounds put mobs into most views
