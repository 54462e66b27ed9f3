"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE).

Only tests, the smoke check and the bench's CPU-baseline leg import this
module.  It wraps ``libcfx_oracle.so`` (the C restatement of the reference's
scalar fp32 policy, see cfx_oracle.c) and, when present, the record producer
built from the reference's own C environment (``_ref/libcfref_env.so``).
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                "craftax.cu_b200"))
from cfx.synth import MAP, OBS, REC, TAIL, init_weights, offsets, synthetic_records  # noqa: E402,F401
from cfx.synth import (CLASSIC_OBS, CLASSIC_REC, classic_init_weights, classic_offsets,  # noqa: E402,F401
                       classic_synthetic_records)

HERE = os.path.dirname(os.path.abspath(__file__))

_lib = None


def build():
    """Compile the oracle (and the reference-derived helpers when the
    reference sources are present)."""
    subprocess.run(["make", "-s", "-C", HERE], check=True)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "libcfx_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.cfxo_param_count.restype = C.c_size_t
        L.cfxo_param_count.argtypes = [C.c_int] * 3
        L.cfxo_expand.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.cfxo_sample.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                  C.c_void_p, C.c_void_p]
        L.cfxo_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_void_p]
        L.cfxo_classic_param_count.restype = C.c_size_t
        L.cfxo_classic_param_count.argtypes = [C.c_int] * 3
        L.cfxo_classic_expand.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.cfxo_classic_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                           C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.cfxo_max_threads.restype = C.c_int
        L.cfxo_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def param_count(H=256, L=2, A=43):
    return int(lib().cfxo_param_count(H, L, A))


def expand(rec):
    rec = np.ascontiguousarray(rec, np.uint8).reshape(-1, REC)
    out = np.empty((rec.shape[0], OBS), np.float32)
    lib().cfxo_expand(_p(rec), _p(out), rec.shape[0])
    return out


def sample(logits, u, A=43):
    logits = np.ascontiguousarray(logits, np.float32)
    n, ld = logits.shape
    u = np.ascontiguousarray(u, np.float32)
    act = np.empty(n, np.int32)
    lp = np.empty(n, np.float32)
    lib().cfxo_sample(_p(logits), ld, A, _p(u), n, _p(act), _p(lp))
    return act, lp


def forward(params, rec, prev_terminals, state, H=256, L=2, A=43, want_h=False,
            want_r_state=False, threads=0):
    """One forward.  state [L][n][H] is updated in place.  Returns logits_av
    [n][A+1] (biases included, value in column A) and optional extras."""
    rec = np.ascontiguousarray(rec, np.uint8).reshape(-1, REC)
    n = rec.shape[0]
    params = np.ascontiguousarray(params, np.float32)
    assert params.size == param_count(H, L, A)
    assert state.dtype == np.float32 and state.shape == (L, n, H) and state.flags.c_contiguous
    pt = None if prev_terminals is None else np.ascontiguousarray(prev_terminals, np.float32)
    lav = np.empty((n, A + 1), np.float32)
    h = np.empty((n, H), np.float32) if want_h else None
    rs = np.empty((L, n, H), np.float32) if want_r_state else None
    if threads:
        lib().cfxo_set_threads(threads)
    lib().cfxo_forward(_p(params), H, L, A, _p(rec), _p(pt), _p(state), n, _p(lav), _p(h), _p(rs))
    out = [lav]
    if want_h:
        out.append(h)
    if want_r_state:
        out.append(rs)
    return out[0] if len(out) == 1 else tuple(out)


def classic_expand(rec):
    rec = np.ascontiguousarray(rec, np.uint8).reshape(-1, CLASSIC_REC)
    out = np.empty((rec.shape[0], CLASSIC_OBS), np.float32)
    lib().cfxo_classic_expand(_p(rec), _p(out), rec.shape[0])
    return out


def classic_forward(params, rec, prev_done, state, H=256, L=3, A=17, want_h_enc=False):
    """Classic-game forward (gather encoder in the reference's order).  prev_done: int8 flags
    or None; state [L][n][H] is updated in place.  Returns logits_av [n][A+1]."""
    rec = np.ascontiguousarray(rec, np.uint8).reshape(-1, CLASSIC_REC)
    n = rec.shape[0]
    params = np.ascontiguousarray(params, np.float32)
    assert params.size == int(lib().cfxo_classic_param_count(H, L, A))
    assert state.dtype == np.float32 and state.shape == (L, n, H) and state.flags.c_contiguous
    pd = None if prev_done is None else np.ascontiguousarray(prev_done, np.int8)
    lav = np.empty((n, A + 1), np.float32)
    he = np.empty((n, H), np.float32) if want_h_enc else None
    lib().cfxo_classic_forward(_p(params), H, L, A, _p(rec), _p(pd), _p(state), n, _p(lav), _p(he))
    return (lav, he) if want_h_enc else lav


def max_threads():
    return int(lib().cfxo_max_threads())


class RefEnv:
    """The reference's C environment (compact-obs build) as a record producer.
    Available only where ``_ref/libcfref_env.so`` has been built."""

    path = os.path.join(HERE, "_ref", "libcfref_env.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.path)

    def __init__(self, n, seed):
        L = C.CDLL(self.path)
        L.refenv_create.restype = C.c_void_p
        L.refenv_create.argtypes = [C.c_int, C.c_ulonglong]
        for f in ("refenv_records", "refenv_terminals", "refenv_rewards", "refenv_actions"):
            getattr(L, f).restype = C.c_void_p
            getattr(L, f).argtypes = [C.c_void_p]
        L.refenv_step_random.argtypes = [C.c_void_p]
        L.refenv_step.argtypes = [C.c_void_p, C.c_void_p]
        L.refenv_destroy.argtypes = [C.c_void_p]
        assert L.refenv_record_size() == REC
        self.L, self.n = L, n
        self.h = L.refenv_create(n, seed)

    def _view(self, ptr, shape, dtype):
        size = int(np.prod(shape)) * np.dtype(dtype).itemsize
        buf = (C.c_char * size).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype).reshape(shape)

    @property
    def records(self):
        return self._view(self.L.refenv_records(self.h), (self.n, REC), np.uint8)

    @property
    def terminals(self):
        return self._view(self.L.refenv_terminals(self.h), (self.n,), np.float32)

    @property
    def rewards(self):
        return self._view(self.L.refenv_rewards(self.h), (self.n,), np.float32)

    @property
    def actions(self):
        return self._view(self.L.refenv_actions(self.h), (self.n,), np.float32)

    def step_random(self):
        self.L.refenv_step_random(self.h)

    def step(self, actions):
        a = np.ascontiguousarray(actions, np.float32)
        self.L.refenv_step(self.h, _p(a))

    def close(self):
        if self.h:
            self.L.refenv_destroy(self.h)
            self.h = None


class RefClassic:
    """The reference's classic-game kernels (expand, gather encoder, MinGRU epilogue, sampler;
    compiled from craftax_classic.cu by oracle/Makefile into ``_ref/libcfref_classic.so``) with
    cuBLAS fp32 products between them.  Runs only on a GPU box."""

    path = os.path.join(HERE, "_ref", "libcfref_classic.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.path)

    def __init__(self):
        L = C.CDLL(self.path)
        L.refcl_expand.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.refcl_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                    C.c_ulonglong, C.c_ulonglong] + [C.c_void_p] * 4
        L.refcl_time_forward.restype = C.c_float
        L.refcl_time_forward.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
        self.L = L
        self.H, self.layers, self.A = L.refcl_hidden(), L.refcl_layers(), L.refcl_actions()
        assert L.refcl_obs() == CLASSIC_OBS and L.refcl_record_bytes() == CLASSIC_REC
        self.param_count = L.refcl_param_count()

    def expand(self, d_rec_ptr, d_out_ptr, n):
        self.L.refcl_expand(d_rec_ptr, d_out_ptr, n)

    def time_forward(self, d_params_ptr, d_rec_ptr, d_prev_done_ptr, d_state_ptr, n, warm=3, iters=10, tf32=1):
        return float(self.L.refcl_time_forward(d_params_ptr, d_rec_ptr, d_prev_done_ptr, d_state_ptr, n,
                                               warm, iters, tf32))

    LOCKSTEP_KEYS = ("max_dlogit", "max_dvalue", "greedy_agreement", "sampled_agreement",
                     "episode_ends", "max_logit", "env_steps")

    def lockstep(self, n, steps, seed, params, precision, tf32=0):
        """Classic rollout on the GPU: the reference's classic env kernels driven by libcfx's
        classic forward (CFX_PREC_* code `precision`), the reference's classic pipeline on the
        same records beside it; returns the device-side comparison figures."""
        if not hasattr(self.L, "refcl_lockstep"):
            raise RuntimeError("reference classic shim built without the lock-step loop")
        self.L.refcl_lockstep.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_void_p, C.c_int, C.c_int,
                                          C.c_void_p]
        p = np.ascontiguousarray(params, np.float32)
        assert p.size == self.param_count
        out = np.zeros(8, np.float64)
        rc = self.L.refcl_lockstep(n, steps, seed, _p(p), precision, tf32, _p(out))
        if rc != 0:
            raise RuntimeError("refcl_lockstep: a cfx call failed (see stderr)")
        return dict(zip(self.LOCKSTEP_KEYS, out.tolist()))

    def forward(self, d_params_ptr, d_rec_ptr, d_prev_done_ptr, d_state_ptr, n, seed, step):
        o = {"logits_av": np.empty((n, self.A + 1), np.float32), "h_enc": np.empty((n, self.H), np.float32),
             "actions": np.empty(n, np.int32), "logprobs": np.empty(n, np.float32)}
        self.L.refcl_forward(d_params_ptr, d_rec_ptr, d_prev_done_ptr, d_state_ptr, n, seed, step,
                             _p(o["logits_av"]), _p(o["h_enc"]), _p(o["actions"]), _p(o["logprobs"]))
        return o


class RefCuda:
    """The reference's own CUDA policy forward (its kernels and cuBLAS wrappers, compiled
    from its sources by oracle/Makefile into ``_ref/libcfref_cuda_l{L}.so``).  Runs only
    on a GPU box; used to pin the oracle and the fused kernel and as the GPU baseline."""

    BF16, TF32, FP32 = 0, 1, 2

    @classmethod
    def path(cls, layers):
        return os.path.join(HERE, "_ref", f"libcfref_cuda_l{layers}.so")

    @classmethod
    def available(cls, layers=2):
        return os.path.exists(cls.path(layers))

    def __init__(self, n, layers=2):
        L = C.CDLL(self.path(layers))
        L.refcu_create.restype = C.c_void_p
        L.refcu_create.argtypes = [C.c_int]
        L.refcu_destroy.argtypes = [C.c_void_p]
        L.refcu_set_weights.argtypes = [C.c_void_p, C.c_void_p]
        L.refcu_get_weights.argtypes = [C.c_void_p, C.c_void_p]
        if hasattr(L, "refcu_save_cfw1"):
            L.refcu_save_cfw1.argtypes = [C.c_void_p, C.c_char_p]
            L.refcu_load_cfw1.argtypes = [C.c_void_p, C.c_char_p]
        L.refcu_set_state.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.refcu_get_state.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.refcu_set_step.argtypes = [C.c_void_p, C.c_ulonglong]
        L.refcu_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_ulonglong,
                                    C.c_void_p] + [C.c_void_p] * 5
        L.refcu_time_forward.restype = C.c_float
        L.refcu_time_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                         C.c_int, C.c_int]
        L.refcu_scalar_set_state.argtypes = [C.c_void_p, C.c_void_p]
        L.refcu_scalar_get_state.argtypes = [C.c_void_p, C.c_void_p]
        L.refcu_scalar_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_ulonglong] + \
            [C.c_void_p] * 4
        assert L.refcu_layers() == layers and L.refcu_hidden() == 256
        self.L, self.n, self.layers, self.H = L, n, layers, 256
        self.h = L.refcu_create(n)

    LOCKSTEP_KEYS = ("max_dlogit", "max_dvalue", "greedy_agreement", "sampled_agreement",
                     "episode_ends", "max_logit", "env_steps")

    @classmethod
    def lockstep(cls, layers, n, steps, seed, params, precision, sync_state=0):
        """Full-game rollout on the GPU: the reference's CUDA env (records written on the device
        by its k_record_obs) driven by libcfx's forward (CFX_PREC_* code `precision`), the
        reference's strict-fp32 cuBLAS pipeline on the same records beside it; returns the
        device-side comparison figures.  libcfx.so must be loaded first (the shim links it)."""
        L = C.CDLL(cls.path(layers))
        if not hasattr(L, "refcu_lockstep"):
            raise RuntimeError("reference shim built without the lock-step loop")
        L.refcu_lockstep.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        p = np.ascontiguousarray(params, np.float32)
        assert p.size == L.refcu_param_count() and L.refcu_layers() == layers
        out = np.zeros(8, np.float64)
        rc = L.refcu_lockstep(n, steps, seed, _p(p), precision, sync_state, _p(out))
        if rc != 0:
            raise RuntimeError("refcu_lockstep: a cfx call failed (see stderr)")
        return dict(zip(cls.LOCKSTEP_KEYS, out.tolist()))

    RECORD_KEYS = ("differing_bytes", "rows_compared", "reference_ms", "cfx_ms", "rows_with_mob",
                   "list_differing_bytes", "skip_differing_bytes")

    @classmethod
    def record_parity(cls, layers, n, steps, fuzz, seed):
        """k_record_obs (craftax_full.cu:9284-9297) beside cfx_record_obs on the reference's CUDA env:
        `steps` steps of random play, then `fuzz` rounds of randomised state; the list variant on
        the last reset list; both kernels timed at n envs.  libcfx.so must be loaded first."""
        L = C.CDLL(cls.path(layers))
        if not hasattr(L, "refcu_record_parity"):
            raise RuntimeError("reference shim built without the record comparison")
        L.refcu_record_parity.argtypes = [C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_void_p]
        out = np.zeros(8, np.float64)
        rc = L.refcu_record_parity(n, steps, fuzz, seed, _p(out))
        if rc != 0:
            raise RuntimeError("refcu_record_parity: a cfx call failed (see stderr)")
        return dict(zip(cls.RECORD_KEYS, out.tolist()))

    @classmethod
    def play(cls, layers, n, steps, seed, load_path, swapped, precision, record_n, record_every,
             frames_path, levels_path):
        """The reference's `play` loop (cu_run_play) and its recorders; swapped != 0 takes the
        policy half of every step from libcfx (which must be loaded first).  Returns the
        frame size in bytes and the byte offset of the action field inside a frame."""
        L = C.CDLL(cls.path(layers))
        if not hasattr(L, "refcu_play"):
            raise RuntimeError("reference shim built without the play loop")
        L.refcu_play.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_char_p, C.c_int, C.c_int, C.c_int,
                                 C.c_int, C.c_int, C.c_char_p, C.c_char_p]
        rc = L.refcu_play(n, steps, seed, os.fsencode(load_path), 1 if swapped else 0, precision, -1,
                          record_n, record_every, os.fsencode(frames_path), os.fsencode(levels_path))
        if rc != 0:
            raise RuntimeError("refcu_play failed (see stderr)")
        return int(L.refcu_frame_bytes()), int(L.refcu_frame_action_offset())

    def set_weights(self, params):
        p = np.ascontiguousarray(params, np.float32)
        assert p.size == self.L.refcu_param_count()
        self.L.refcu_set_weights(self.h, _p(p))

    def get_weights(self):
        p = np.empty(self.L.refcu_param_count(), np.float32)
        self.L.refcu_get_weights(self.h, _p(p))
        return p

    def save_cfw1(self, path):
        """The reference's cu_save_weights on its current arena."""
        self.L.refcu_save_cfw1(self.h, os.fsencode(path))

    def load_cfw1(self, path):
        """The reference's cu_load_weights; returns its status (0 = loaded)."""
        return int(self.L.refcu_load_cfw1(self.h, os.fsencode(path)))

    def set_state(self, mode, state):
        s = np.ascontiguousarray(state, np.float32)
        assert s.shape == (self.layers, self.n, self.H)
        self.L.refcu_set_state(self.h, mode, _p(s))

    def get_state(self, mode):
        s = np.empty((self.layers, self.n, self.H), np.float32)
        self.L.refcu_get_state(self.h, mode, _p(s))
        return s

    def set_step(self, step):
        self.L.refcu_set_step(self.h, step)

    def forward(self, mode, d_rec_ptr, d_prev_terminals_ptr, seed):
        """Device pointers in; returns dict with logits_av (biases NOT included, as the
        reference stores them), h3, actions, logprobs, values (host arrays)."""
        n = self.n
        o = {"logits_nobias": np.empty((n, 44), np.float32), "h3": np.empty((n, self.H), np.float32),
             "actions": np.empty(n, np.int32), "logprobs": np.empty(n, np.float32),
             "values": np.empty(n, np.float32)}
        self.L.refcu_forward(self.h, mode, d_rec_ptr, d_prev_terminals_ptr, seed, None,
                             _p(o["logits_nobias"]), _p(o["h3"]), _p(o["actions"]),
                             _p(o["logprobs"]), _p(o["values"]))
        return o

    def time_forward(self, mode, d_rec_ptr, d_prev_terminals_ptr, warm=3, iters=10, graph=1):
        return float(self.L.refcu_time_forward(self.h, mode, d_rec_ptr, d_prev_terminals_ptr,
                                               warm, iters, graph))

    def scalar_set_state(self, state):
        s = np.ascontiguousarray(state, np.float32)
        self.L.refcu_scalar_set_state(self.h, _p(s))

    def scalar_get_state(self):
        s = np.empty((self.layers, self.n, self.H), np.float32)
        self.L.refcu_scalar_get_state(self.h, _p(s))
        return s

    def scalar_forward(self, d_rec_ptr, d_prev_terminals_ptr, seed):
        n = self.n
        o = {"h3": np.empty((n, self.H), np.float32), "actions": np.empty(n, np.int32),
             "logprobs": np.empty(n, np.float32), "values": np.empty(n, np.float32)}
        self.L.refcu_scalar_forward(self.h, d_rec_ptr, d_prev_terminals_ptr, seed, _p(o["h3"]),
                                    _p(o["actions"]), _p(o["logprobs"]), _p(o["values"]))
        return o

    def close(self):
        if self.h:
            self.L.refcu_destroy(self.h)
            self.h = None
