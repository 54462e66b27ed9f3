"""ctypes binding of libcfx.so -- the host-side mirror of the reference's
policy interface (CuPolicy + cu_rollout_step's forward half, craftax_full.cu:
11758-12048) for Python callers, tests and the benchmark.

There is no fallback: importing works anywhere (the library only needs the CUDA
runtime it links statically), but every compute call needs a B200 and fails
loudly otherwise.
"""
import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# CFX_LIB (environment) names another build of the same library, e.g. a debug build
LIB_PATH = os.environ.get("CFX_LIB") or os.path.join(PKG, "libcfx.so")

OBS, MAP, TAIL, REC = 843, 792, 51, 996
CLASSIC_OBS, CLASSIC_REC = 1345, 148
PREC_FP32, PREC_F16, PREC_BF16, PREC_TF32 = 0, 1, 2, 3
PREC_NAMES = {"fp32": 0, "f16": 1, "bf16": 2, "tf32": 3}
OK, ERR_INVALID, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_IO, ERR_UNSUPPORTED = 0, 1, 2, 3, 4, 5


class CfxError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"cfx status {code}: {msg}")
        self.code = code


class ForwardIO(C.Structure):
    _fields_ = [("records", C.c_void_p), ("prev_terminals", C.c_void_p),
                ("uniforms", C.c_void_p), ("env_actions", C.c_void_p),
                ("actions", C.c_void_p), ("logprobs", C.c_void_p), ("values", C.c_void_p),
                ("logits_av", C.c_void_p), ("r_state", C.c_void_p), ("seed", C.c_uint64),
                ("env_offset", C.c_uint64), ("bump_step", C.c_int), ("r_state_bf16", C.c_int)]


# the SoA fields of cfx_env_view, in the order of include/cfx.h: (name, numpy dtype, elements per env)
ENV_VIEW_FIELDS = (
    ("player_position", "i4", 2), ("player_level", "i4", 1), ("player_direction", "i4", 1),
    ("player_health", "f4", 1), ("player_food", "i4", 1), ("player_drink", "i4", 1), ("player_energy", "i4", 1),
    ("player_mana", "i4", 1), ("is_sleeping", "u1", 1), ("is_resting", "u1", 1), ("player_xp", "i4", 1),
    ("player_dexterity", "i4", 1), ("player_strength", "i4", 1), ("player_intelligence", "i4", 1),
    ("inv_wood", "i4", 1), ("inv_stone", "i4", 1), ("inv_coal", "i4", 1), ("inv_iron", "i4", 1),
    ("inv_diamond", "i4", 1), ("inv_sapling", "i4", 1), ("inv_pickaxe", "i4", 1), ("inv_sword", "i4", 1),
    ("inv_bow", "i4", 1), ("inv_arrows", "i4", 1), ("inv_torches", "i4", 1), ("inv_ruby", "i4", 1),
    ("inv_sapphire", "i4", 1), ("inv_books", "i4", 1), ("inv_armour", "i4", 4), ("inv_potions", "i4", 6),
    ("learned_spells", "u1", 2), ("sword_enchantment", "i4", 1), ("bow_enchantment", "i4", 1),
    ("armour_enchantments", "i4", 4), ("boss_timesteps_to_spawn_this_round", "i4", 1), ("light_level", "f4", 1),
    ("monsters_killed", "i4", 9), ("mob_position", "i4", 270), ("mob_mask", "u1", 135), ("mob_type_id", "i4", 135),
)
ENV_VIEW_MAPS = ("map", "item_map", "light_map")   # uint8 [9][48][48] inside every env's block
ENV_MAP_BYTES = 9 * 48 * 48


class EnvView(C.Structure):
    """cfx_env_view of include/cfx.h."""
    _fields_ = [("num_envs", C.c_int32), ("state_base", C.c_void_p), ("state_stride", C.c_uint64),
                ("map_offset", C.c_uint64), ("item_map_offset", C.c_uint64), ("light_map_offset", C.c_uint64)] + \
               [(name, C.c_void_p) for name, _, _ in ENV_VIEW_FIELDS]


_SIGS = {
    "cfx_param_count": (C.c_size_t, [C.c_int] * 3),
    "cfx_policy_create": (C.c_int, [C.POINTER(C.c_void_p)] + [C.c_int] * 6),
    "cfx_policy_destroy": (C.c_int, [C.c_void_p]),
    "cfx_policy_set_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]),
    "cfx_policy_get_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "cfx_policy_init_weights": (C.c_int, [C.c_void_p, C.c_uint64]),
    "cfx_policy_save_cfw1": (C.c_int, [C.c_void_p, C.c_char_p]),
    "cfx_policy_load_cfw1": (C.c_int, [C.c_void_p, C.c_char_p]),
    "cfx_policy_set_precision": (C.c_int, [C.c_void_p, C.c_int]),
    "cfx_policy_get_precision": (C.c_int, [C.c_void_p]),
    "cfx_policy_state": (C.c_void_p, [C.c_void_p]),
    "cfx_policy_reset_state": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cfx_policy_set_step": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "cfx_policy_get_step": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "cfx_policy_bump_step": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cfx_policy_stream": (C.c_void_p, [C.c_void_p]),
    "cfx_policy_last_launches": (C.c_int, [C.c_void_p]),
    "cfx_policy_forward": (C.c_int, [C.c_void_p, C.POINTER(ForwardIO), C.c_void_p]),
    "cfx_policy_forward_host": (C.c_int, [C.c_void_p, C.POINTER(ForwardIO)]),
    "cfx_policy_check": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cfx_selftest_wait_timeout": (C.c_int, [C.c_int, C.c_uint]),
    "cfx_strict_forward_static": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_void_p, C.POINTER(ForwardIO), C.c_void_p, C.c_void_p]),
    "cfx_classic_param_count": (C.c_size_t, [C.c_int] * 3),
    "cfx_policy_create_classic": (C.c_int, [C.POINTER(C.c_void_p)] + [C.c_int] * 6),
    "cfx_classic_expand_obs": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "cfx_classic_done_to_terminals": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "cfx_expand_obs": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    # record write from the reference's device state (the view is a cfx_env_view filled in C)
    "cfx_record_obs": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "cfx_record_obs_list": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                      C.c_void_p]),
    "cfx_classic_record_obs": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "cfx_sample_actions": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "cfx_philox_uniforms": (C.c_int, [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int,
                                      C.c_void_p, C.c_void_p]),
    "cfx_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "cfx_device_name": (C.c_int, [C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_int),
                                  C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "cfx_device_alloc": (C.c_int, [C.c_int, C.POINTER(C.c_void_p), C.c_size_t]),
    "cfx_device_free": (C.c_int, [C.c_int, C.c_void_p]),
    "cfx_host_alloc_pinned": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "cfx_host_free_pinned": (C.c_int, [C.c_void_p]),
    "cfx_memcpy_h2d": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cfx_memcpy_d2h": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cfx_memset": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "cfx_stream_sync": (C.c_int, [C.c_int, C.c_void_p]),
    "cfx_timer_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "cfx_timer_destroy": (C.c_int, [C.c_void_p]),
    "cfx_timer_start": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cfx_timer_stop": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cfx_timer_elapsed_ms": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "cfx_last_error": (C.c_char_p, []),
    "cfx_version": (C.c_char_p, []),
}

_lib = None


def declared_symbols():
    """Names of every entry point declared in include/cfx.h that this binding knows."""
    return sorted(_SIGS)


def lib():
    """Loads libcfx.so; raises when it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CfxError(-1, f"{LIB_PATH} is missing: run `python craftax.cu_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            if not hasattr(L, name):
                continue  # optional entry points are resolved on use
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise CfxError(rc, lib().cfx_last_error().decode())


def device_count():
    n = C.c_int(0)
    rc = lib().cfx_device_count(C.byref(n))
    return n.value if rc == 0 else 0


def device_info(device=0):
    buf = C.create_string_buffer(256)
    sm, ma, mi = C.c_int(), C.c_int(), C.c_int()
    check(lib().cfx_device_name(device, buf, 256, C.byref(sm), C.byref(ma), C.byref(mi)))
    return {"name": buf.value.decode(), "sms": sm.value, "cc": (ma.value, mi.value)}


class DeviceBuffer:
    """A typed device allocation with numpy-shaped host transfers."""

    def __init__(self, shape, dtype, device=0, zero=False):
        self.shape = tuple(np.atleast_1d(shape).tolist()) if not isinstance(shape, tuple) else shape
        self.dtype = np.dtype(dtype)
        self.device = device
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        p = C.c_void_p()
        check(lib().cfx_device_alloc(device, C.byref(p), self.nbytes))
        self.ptr = p.value
        if zero:
            self.fill(0)

    @classmethod
    def from_host(cls, arr, device=0):
        arr = np.ascontiguousarray(arr)
        b = cls(arr.shape, arr.dtype, device)
        b.upload(arr)
        return b

    def upload(self, arr, stream=None):
        arr = np.ascontiguousarray(arr, self.dtype)
        assert arr.nbytes == self.nbytes, (arr.shape, self.shape)
        check(lib().cfx_memcpy_h2d(self.device, self.ptr, arr.ctypes.data, self.nbytes, stream))
        check(lib().cfx_stream_sync(self.device, stream))

    def download(self, stream=None):
        out = np.empty(self.shape, self.dtype)
        check(lib().cfx_memcpy_d2h(self.device, out.ctypes.data, self.ptr, self.nbytes, stream))
        check(lib().cfx_stream_sync(self.device, stream))
        return out

    def fill(self, byte, stream=None):
        check(lib().cfx_memset(self.device, self.ptr, byte, self.nbytes, stream))
        check(lib().cfx_stream_sync(self.device, stream))

    def free(self):
        if self.ptr:
            lib().cfx_device_free(self.device, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PinnedBuffer:
    """Page-locked host array (numpy view) for full-speed host<->device copies."""

    def __init__(self, shape, dtype):
        self.dtype = np.dtype(dtype)
        self.shape = shape if isinstance(shape, tuple) else (int(shape),)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        p = C.c_void_p()
        check(lib().cfx_host_alloc_pinned(C.byref(p), self.nbytes))
        self.ptr = p.value
        buf = (C.c_char * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype).reshape(self.shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib().cfx_host_free_pinned(self.ptr)
            self.ptr = None


class Timer:
    def __init__(self, device=0):
        t = C.c_void_p()
        check(lib().cfx_timer_create(device, C.byref(t)))
        self.t = t.value

    def start(self, stream=None):
        check(lib().cfx_timer_start(self.t, stream))

    def stop(self, stream=None):
        check(lib().cfx_timer_stop(self.t, stream))

    def elapsed_ms(self):
        ms = C.c_float()
        check(lib().cfx_timer_elapsed_ms(self.t, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            lib().cfx_timer_destroy(self.t)
        except Exception:
            pass


class Policy:
    """Mirror of the reference's CuPolicy for one GPU: weights, recurrent state,
    step counter, and the batched forward."""

    def __init__(self, n, hidden=256, layers=2, actions=43, precision="fp32", device=0, game="full"):
        self.n, self.H, self.L, self.A, self.device = n, hidden, layers, actions, device
        self.game = game
        self.rec_bytes = CLASSIC_REC if game == "classic" else REC
        prec = PREC_NAMES[precision] if isinstance(precision, str) else int(precision)
        h = C.c_void_p()
        if game == "classic":     # 148-byte records, 1345 features
            check(lib().cfx_policy_create_classic(C.byref(h), device, n, hidden, layers, actions, prec))
        else:
            check(lib().cfx_policy_create(C.byref(h), device, n, hidden, layers, actions, prec))
        self.h = h.value
        self.stream = lib().cfx_policy_stream(self.h)
        self._out = None

    # -- weights ---------------------------------------------------------
    @property
    def param_count(self):
        f = lib().cfx_classic_param_count if self.game == "classic" else lib().cfx_param_count
        return int(f(self.H, self.L, self.A))

    def set_weights(self, arena):
        a = np.ascontiguousarray(arena, np.float32)
        check(lib().cfx_policy_set_weights(self.h, a.ctypes.data, a.size, 0))

    def get_weights(self):
        a = np.empty(self.param_count, np.float32)
        check(lib().cfx_policy_get_weights(self.h, a.ctypes.data, a.size))
        return a

    def init_weights(self, seed=1234):
        check(lib().cfx_policy_init_weights(self.h, seed))

    def save(self, path):
        check(lib().cfx_policy_save_cfw1(self.h, os.fsencode(path)))

    def load(self, path):
        check(lib().cfx_policy_load_cfw1(self.h, os.fsencode(path)))

    def set_precision(self, precision):
        prec = PREC_NAMES[precision] if isinstance(precision, str) else int(precision)
        check(lib().cfx_policy_set_precision(self.h, prec))

    # -- state -----------------------------------------------------------
    def reset_state(self):
        check(lib().cfx_policy_reset_state(self.h, None))
        self.sync()

    def get_state(self):
        out = np.empty((self.L, self.n, self.H), np.float32)
        check(lib().cfx_memcpy_d2h(self.device, out.ctypes.data, lib().cfx_policy_state(self.h),
                                   out.nbytes, self.stream))
        self.sync()
        return out

    def set_state(self, state):
        s = np.ascontiguousarray(state, np.float32)
        assert s.shape == (self.L, self.n, self.H)
        check(lib().cfx_memcpy_h2d(self.device, lib().cfx_policy_state(self.h), s.ctypes.data,
                                   s.nbytes, self.stream))
        self.sync()

    @property
    def step(self):
        v = C.c_uint64()
        check(lib().cfx_policy_get_step(self.h, C.byref(v)))
        return v.value

    @step.setter
    def step(self, v):
        check(lib().cfx_policy_set_step(self.h, int(v), None))

    def sync(self):
        check(lib().cfx_stream_sync(self.device, self.stream))

    def check(self, stream=None):
        """Synchronise and raise if a device-side bounded wait gave up."""
        check(lib().cfx_policy_check(self.h, stream))

    @property
    def last_launches(self):
        return lib().cfx_policy_last_launches(self.h)

    # -- forward ---------------------------------------------------------
    def forward_device(self, records, prev_terminals=None, uniforms=None, *, env_actions=None,
                       actions, logprobs=None, values=None, logits_av=None, r_state=None,
                       seed=0, env_offset=0, bump_step=False, stream=None, r_state_bf16=False):
        """Device-pointer forward (arguments are DeviceBuffer or None); asynchronous.
        `r_state` holds fp32 [L][n][H], or bf16 of the same shape with r_state_bf16."""
        def p(b):
            return None if b is None else b.ptr
        io = ForwardIO(p(records), p(prev_terminals), p(uniforms), p(env_actions), p(actions),
                       p(logprobs), p(values), p(logits_av), p(r_state), seed, env_offset,
                       1 if bump_step else 0, 1 if r_state_bf16 else 0)
        check(lib().cfx_policy_forward(self.h, C.byref(io), stream))

    def forward_host(self, records, prev_terminals=None, uniforms=None, *, seed=0, env_offset=0,
                     bump_step=False, want_logits=True, want_r_state=False, out=None):
        """Host-buffer forward through cfx_policy_forward_host; returns a dict of numpy
        arrays.  `out` may hold preallocated (pinned) arrays to reuse.  want_r_state: True for
        the fp32 record of the post-zero input state, "bf16" for the bf16 record (returned as
        the uint16 bit patterns)."""
        n, A = self.n, self.A
        rec = np.ascontiguousarray(records, np.uint8)
        assert rec.size == n * self.rec_bytes
        o = out if out is not None else {}
        o.setdefault("env_actions", np.empty(n, np.float32))
        o.setdefault("actions", np.empty(n, np.int32))
        o.setdefault("logprobs", np.empty(n, np.float32))
        o.setdefault("values", np.empty(n, np.float32))
        if want_logits:
            o.setdefault("logits_av", np.empty((n, A + 1), np.float32))
        if want_r_state:
            o.setdefault("r_state", np.empty((self.L, n, self.H),
                                             np.uint16 if want_r_state == "bf16" else np.float32))
        pt = None if prev_terminals is None else np.ascontiguousarray(prev_terminals, np.float32)
        u = None if uniforms is None else np.ascontiguousarray(uniforms, np.float32)

        def hp(a):
            return None if a is None else a.ctypes.data
        io = ForwardIO(hp(rec), hp(pt), hp(u), hp(o["env_actions"]), hp(o["actions"]),
                       hp(o["logprobs"]), hp(o["values"]), hp(o.get("logits_av")),
                       hp(o.get("r_state")), seed, env_offset, 1 if bump_step else 0,
                       1 if want_r_state == "bf16" else 0)
        check(lib().cfx_policy_forward_host(self.h, C.byref(io)))
        return o

    def close(self):
        if self.h:
            lib().cfx_policy_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def expand_obs(records, device=0):
    """records uint8 [n][996] (host) -> fp32 features [n][843] via the device kernel."""
    rec = np.ascontiguousarray(records, np.uint8).reshape(-1, REC)
    n = rec.shape[0]
    d_rec = DeviceBuffer.from_host(rec, device)
    d_out = DeviceBuffer((n, OBS), np.float32, device)
    check(lib().cfx_expand_obs(device, d_rec.ptr, d_out.ptr, n, None))
    return d_out.download()


def classic_expand_obs(records, device=0):
    """classic records uint8 [n][148] (host) -> fp32 features [n][1345] via the device kernel."""
    rec = np.ascontiguousarray(records, np.uint8).reshape(-1, CLASSIC_REC)
    n = rec.shape[0]
    d_rec = DeviceBuffer.from_host(rec, device)
    d_out = DeviceBuffer((n, CLASSIC_OBS), np.float32, device)
    check(lib().cfx_classic_expand_obs(device, d_rec.ptr, d_out.ptr, n, None))
    return d_out.download()


def classic_done_to_terminals(done, device=0):
    d = np.ascontiguousarray(done, np.int8)
    d_in = DeviceBuffer.from_host(d, device)
    d_out = DeviceBuffer((d.size,), np.float32, device)
    check(lib().cfx_classic_done_to_terminals(device, d_in.ptr, d_out.ptr, d.size, None))
    return d_out.download()


def sample_actions(logits, uniforms, num_actions=43, device=0):
    lg = np.ascontiguousarray(logits, np.float32)
    n, ld = lg.shape
    d_l = DeviceBuffer.from_host(lg, device)
    d_u = DeviceBuffer.from_host(np.ascontiguousarray(uniforms, np.float32), device)
    d_a = DeviceBuffer((n,), np.int32, device)
    d_p = DeviceBuffer((n,), np.float32, device)
    check(lib().cfx_sample_actions(device, d_l.ptr, ld, num_actions, d_u.ptr, n, d_a.ptr, d_p.ptr, None))
    return d_a.download(), d_p.download()


def env_view_from_state(state, device=0):
    """Uploads a state dict (one [count][n] array per field of ENV_VIEW_FIELDS, one
    [n][9][48][48] byte array per map) and returns (EnvView, buffers to keep alive).  The per-env
    block holds the three maps back to back."""
    n = state["player_level"].shape[1]
    keep, view = [], EnvView()
    view.num_envs = n
    blocks = np.ascontiguousarray(np.stack([state[m].reshape(n, ENV_MAP_BYTES) for m in ENV_VIEW_MAPS], axis=1))
    d_blocks = DeviceBuffer.from_host(blocks, device)
    keep.append(d_blocks)
    view.state_base, view.state_stride = d_blocks.ptr, 3 * ENV_MAP_BYTES
    view.map_offset, view.item_map_offset, view.light_map_offset = 0, ENV_MAP_BYTES, 2 * ENV_MAP_BYTES
    for name, dt, cnt in ENV_VIEW_FIELDS:
        a = np.ascontiguousarray(state[name], np.dtype(dt))
        assert a.shape == (cnt, n), (name, a.shape)
        b = DeviceBuffer.from_host(a, device)
        keep.append(b)
        setattr(view, name, b.ptr)
    return view, keep


def env_state_from_view(view, device=0):
    """The reverse: downloads every field and the three maps behind an EnvView (device pointers)
    into a state dict."""
    n = view.num_envs
    L = lib()

    def fetch(ptr, shape, dt):
        out = np.empty(shape, np.dtype(dt))
        check(L.cfx_memcpy_d2h(device, out.ctypes.data, ptr, out.nbytes, None))
        check(L.cfx_stream_sync(device, None))
        return out
    st = {name: fetch(getattr(view, name), (cnt, n), dt) for name, dt, cnt in ENV_VIEW_FIELDS}
    blocks = fetch(view.state_base, (n, view.state_stride), "u1")
    for m, off in zip(ENV_VIEW_MAPS, (view.map_offset, view.item_map_offset, view.light_map_offset)):
        st[m] = blocks[:, off:off + ENV_MAP_BYTES].reshape(n, 9, 48, 48).copy()
    return st


def record_obs(view, d_records, n=None, skip=None, device=0, stream=None):
    """cfx_record_obs: the [n][996] records of the envs behind `view` into a DeviceBuffer."""
    check(lib().cfx_record_obs(device, C.byref(view), d_records.ptr, view.num_envs if n is None else n,
                               None if skip is None else skip.ptr, stream))


def record_obs_list(view, d_records, d_list, list_stride, d_count, device=0, stream=None):
    """cfx_record_obs_list: the envs named by the first int32 of every list entry."""
    check(lib().cfx_record_obs_list(device, C.byref(view), d_records.ptr, d_list.ptr, list_stride, d_count.ptr,
                                    stream))


def philox_uniforms(seed, env_offset, step, n, device=0):
    d_u = DeviceBuffer((n,), np.float32, device)
    check(lib().cfx_philox_uniforms(device, seed, env_offset, step, n, d_u.ptr, None))
    return d_u.download()
