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


# ---- record write (reference cf_record_env_warp, craftax_full.cu:9180-9269, scalar tail
# craftax_encode_scalar_observation_tail_at :2429-2487): a numpy restatement over a dict of
# arrays, one entry per SoA field of CF_SOA_FIELDS (:620-690) that the record reads, shaped
# [count][n] like the reference's device layout, plus the three byte maps [n][9][48][48].
RECORD_FIELDS = {   # name: (dtype, count)
    "player_position": (np.int32, 2), "player_level": (np.int32, 1), "player_direction": (np.int32, 1),
    "player_health": (np.float32, 1), "player_food": (np.int32, 1), "player_drink": (np.int32, 1),
    "player_energy": (np.int32, 1), "player_mana": (np.int32, 1), "is_sleeping": (np.uint8, 1),
    "is_resting": (np.uint8, 1), "player_xp": (np.int32, 1), "player_dexterity": (np.int32, 1),
    "player_strength": (np.int32, 1), "player_intelligence": (np.int32, 1), "inv_wood": (np.int32, 1),
    "inv_stone": (np.int32, 1), "inv_coal": (np.int32, 1), "inv_iron": (np.int32, 1),
    "inv_diamond": (np.int32, 1), "inv_sapling": (np.int32, 1), "inv_pickaxe": (np.int32, 1),
    "inv_sword": (np.int32, 1), "inv_bow": (np.int32, 1), "inv_arrows": (np.int32, 1),
    "inv_torches": (np.int32, 1), "inv_ruby": (np.int32, 1), "inv_sapphire": (np.int32, 1),
    "inv_books": (np.int32, 1), "inv_armour": (np.int32, 4), "inv_potions": (np.int32, 6),
    "learned_spells": (np.uint8, 2), "sword_enchantment": (np.int32, 1), "bow_enchantment": (np.int32, 1),
    "armour_enchantments": (np.int32, 4), "boss_timesteps_to_spawn_this_round": (np.int32, 1),
    "light_level": (np.float32, 1), "monsters_killed": (np.int32, 9), "mob_position": (np.int32, 270),
    "mob_mask": (np.uint8, 135), "mob_type_id": (np.int32, 135),
}
RECORD_MAPS = ("map", "item_map", "light_map")   # uint8 [n][9][48][48] each


def jax_index(i, size):
    """craftax_wg_jax_index (:1963-1975): a negative index wraps once, then the index is clamped."""
    i = np.where(i < 0, i + size, i)
    return np.clip(i, 0, size - 1)


def record_from_state(st):
    """The [n][996] records of a state dict (RECORD_FIELDS + RECORD_MAPS)."""
    n = st["player_level"].shape[1]
    rec = np.zeros((n, 996), np.uint8)
    tail = np.zeros((n, 51), np.float32)
    f32 = np.float32
    level = st["player_level"][0].astype(np.int64)
    mob_level = jax_index(level, 9)

    def sq10(x):
        return np.sqrt(x.astype(f32)) * f32(1.0 / 10.0)
    k = 0
    for name in ("inv_wood", "inv_stone", "inv_coal", "inv_iron", "inv_diamond", "inv_sapphire", "inv_ruby",
                 "inv_sapling", "inv_torches", "inv_arrows"):
        tail[:, k] = sq10(st[name][0]); k += 1
    tail[:, k] = st["inv_books"][0].astype(f32) * f32(0.5); k += 1
    tail[:, k] = st["inv_pickaxe"][0].astype(f32) * f32(0.25); k += 1
    tail[:, k] = st["inv_sword"][0].astype(f32) * f32(0.25); k += 1
    for name in ("sword_enchantment", "bow_enchantment", "inv_bow"):
        tail[:, k] = st[name][0].astype(f32); k += 1
    for i in range(6):
        tail[:, k] = sq10(st["inv_potions"][i]); k += 1
    tail[:, k] = st["player_health"][0] * f32(1.0 / 10.0); k += 1
    for name in ("player_food", "player_drink", "player_energy", "player_mana", "player_xp",
                 "player_dexterity", "player_strength", "player_intelligence"):
        tail[:, k] = st[name][0].astype(f32) * f32(1.0 / 10.0); k += 1
    for i in range(4):
        tail[:, k] = (st["player_direction"][0] - 1 == i); k += 1
    for i in range(4):
        tail[:, k] = st["inv_armour"][i].astype(f32) * f32(0.5); k += 1
    for i in range(4):
        tail[:, k] = st["armour_enchantments"][i].astype(f32); k += 1
    tail[:, k] = st["light_level"][0]; k += 1
    for a in (st["is_sleeping"][0], st["is_resting"][0], st["learned_spells"][0], st["learned_spells"][1]):
        tail[:, k] = a != 0; k += 1
    tail[:, k] = st["player_level"][0].astype(f32) * f32(1.0 / 10.0); k += 1
    env = np.arange(n)
    tail[:, k] = st["monsters_killed"][np.clip(level, 0, 8), env] >= 8; k += 1   # level is in [0, 9) in every env state

    def midx(c, lvl, i):
        return (c * 9 + lvl) * 3 + i
    alive = np.zeros(n, bool)
    for c, slots in ((0, 3), (2, 2)):   # craftax_wg_is_boss_vulnerable (:1988-2003)
        for i in range(slots):
            alive |= st["mob_mask"][midx(c, mob_level, i), env] != 0
    tail[:, k] = ~alive & (st["boss_timesteps_to_spawn_this_round"][0] <= 0); k += 1
    assert k == 51
    rec[:, 792:] = tail.view(np.uint8).reshape(n, 204)

    top = st["player_position"][0].astype(np.int64) - 4
    left = st["player_position"][1].astype(np.int64) - 5
    cells = np.zeros((n, 9, 11, 8), np.uint8)
    rr = top[:, None, None] + np.arange(9)[None, :, None]
    cc = left[:, None, None] + np.arange(11)[None, None, :]
    inb = (rr >= 0) & (rr < 48) & (cc >= 0) & (cc < 48)
    rc, ccl = np.clip(rr, 0, 47), np.clip(cc, 0, 47)
    e3 = env[:, None, None]
    lv3 = np.clip(level, 0, 8)[:, None, None]
    lit = inb & (st["light_map"][e3, lv3, rc, ccl] > 12)
    cells[..., 0] = np.where(lit, st["map"][e3, lv3, rc, ccl], 0)
    cells[..., 1] = np.where(lit, (st["item_map"][e3, lv3, rc, ccl].astype(np.int32) + 1) & 255, 0)
    cells[..., 2] = lit
    # mobs in class-major, slot-minor order: a later slot of a class overwrites an earlier one (:9195-9236)
    for c in range(5):
        for i in range(2 if c == 2 else 3):
            idx = midx(c, mob_level, i)
            t = st["mob_type_id"][idx, env]
            m = st["mob_mask"][idx, env] != 0
            mr = st["mob_position"][idx * 2, env].astype(np.int64)
            mc = st["mob_position"][idx * 2 + 1, env].astype(np.int64)
            lr, lc = mr - top, mc - left
            ok = (t >= 0) & (t < 8) & m & (lr >= 0) & (lr < 9) & (lc >= 0) & (lc < 11) & \
                 (mr >= 0) & (mr < 48) & (mc >= 0) & (mc < 48)
            okl = ok & (st["light_map"][env, mob_level, np.clip(mr, 0, 47), np.clip(mc, 0, 47)] > 12)
            sel = np.nonzero(okl)[0]
            cells[sel, lr[sel], lc[sel], 3 + c] = (t[sel] + 1).astype(np.uint8)
    rec[:, :792] = cells.reshape(n, 792)
    return rec


def synthetic_env_state(n, seed=0):
    """A random state dict with the value ranges of the game: players anywhere on the map, mobs
    of every class and slot near the player (some off the view, off the map, unlit, masked out or
    with a type id out of range), random blocks, items and light around the player."""
    rng = np.random.default_rng(seed)
    st = {}
    for name, (dt, cnt) in RECORD_FIELDS.items():
        st[name] = np.zeros((cnt, n), dt)
    st["player_level"][0] = rng.integers(0, 9, n)
    st["player_position"][:] = rng.integers(0, 48, (2, n))
    st["player_direction"][0] = rng.integers(0, 6, n)
    st["player_health"][0] = rng.integers(0, 100, n).astype(np.float32) * np.float32(0.125)
    for name in ("player_food", "player_drink", "player_energy", "player_mana", "player_xp", "player_dexterity",
                 "player_strength", "player_intelligence", "inv_pickaxe", "inv_sword", "inv_bow", "inv_books",
                 "sword_enchantment", "bow_enchantment"):
        st[name][0] = rng.integers(0, 10, n)
    for name in ("inv_wood", "inv_stone", "inv_coal", "inv_iron", "inv_diamond", "inv_sapling", "inv_arrows",
                 "inv_torches", "inv_ruby", "inv_sapphire"):
        st[name][0] = rng.integers(0, 100, n)
    st["inv_armour"][:] = rng.integers(0, 3, (4, n))
    st["armour_enchantments"][:] = rng.integers(0, 3, (4, n))
    st["inv_potions"][:] = rng.integers(0, 30, (6, n))
    for name in ("is_sleeping", "is_resting"):
        st[name][0] = rng.integers(0, 2, n)
    st["learned_spells"][:] = rng.integers(0, 2, (2, n))
    st["boss_timesteps_to_spawn_this_round"][0] = rng.integers(-2, 3, n)
    st["light_level"][0] = rng.integers(0, 1000, n).astype(np.float32) * np.float32(0.001)
    st["monsters_killed"][:] = rng.integers(0, 16, (9, n))
    st["mob_type_id"][:] = rng.integers(-1, 9, (135, n))
    st["mob_mask"][:] = rng.integers(0, 4, (135, n)) != 0
    pos = np.empty((135, 2, n), np.int64)
    pos[:, 0] = st["player_position"][0][None, :] + rng.integers(-6, 7, (135, n))
    pos[:, 1] = st["player_position"][1][None, :] + rng.integers(-7, 8, (135, n))
    st["mob_position"][:] = pos.reshape(270, n)
    st["map"] = rng.integers(0, 40, (n, 9, 48, 48)).astype(np.uint8)
    st["item_map"] = rng.integers(0, 6, (n, 9, 48, 48)).astype(np.uint8)
    st["light_map"] = rng.integers(0, 26, (n, 9, 48, 48)).astype(np.uint8)
    return st


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

    def rollout_sps(self, n, steps, seed, params, mode, precision):
        """Whole classic rollouts on the GPU, env-steps per second: mode 0 the reference's own step
        (main_classic.cu Rollout::step), 1 with the policy half from libcfx, 2 with the record
        write from libcfx too."""
        self.L.refcl_rollout_sps.restype = C.c_double
        self.L.refcl_rollout_sps.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_void_p, C.c_int, C.c_int]
        p = np.ascontiguousarray(params, np.float32)
        assert p.size == self.param_count
        v = self.L.refcl_rollout_sps(n, steps, seed, _p(p), mode, precision)
        if v <= 0:
            raise RuntimeError("refcl_rollout_sps: a cfx call failed (see stderr)")
        return v

    RECORD_KEYS = ("differing_bytes", "rows_compared", "reference_ms", "cfx_ms", "rows_with_mob", "episode_ends")

    def record_parity(self, n, steps, seed):
        """record_obs_kernel (craftax_classic.cu:1884-1890) beside cfx_classic_record_obs on the
        reference's classic CUDA env over `steps` steps of random play with auto-reset; both
        kernels timed at n envs."""
        if not hasattr(self.L, "refcl_record_parity"):
            raise RuntimeError("reference classic shim built without the record comparison")
        self.L.refcl_record_parity.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_void_p]
        out = np.zeros(8, np.float64)
        rc = self.L.refcl_record_parity(n, steps, seed, _p(out))
        if rc != 0:
            raise RuntimeError("refcl_record_parity: a cfx call failed (see stderr)")
        return dict(zip(self.RECORD_KEYS, out.tolist()))

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
    def record_session(cls, layers, n, steps, fuzz, seed, view):
        """Plays the reference's CUDA env (`steps` random steps, `fuzz` rounds of randomised
        state), returns the records its k_record_obs writes and fills `view` (a ctypes mirror of
        cfx_env_view) with pointers to the live state; call record_session_close when done."""
        L = C.CDLL(cls.path(layers))
        L.refcu_record_session_open.argtypes = [C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_void_p, C.c_size_t,
                                                C.c_void_p]
        rec = np.empty((n, 996), np.uint8)
        rc = L.refcu_record_session_open(n, steps, fuzz, seed, C.addressof(view), C.sizeof(view), _p(rec))
        if rc != 0:
            raise RuntimeError("refcu_record_session_open failed (a session is open, or the view's size differs)")
        return rec

    @classmethod
    def record_session_close(cls, layers):
        C.CDLL(cls.path(layers)).refcu_record_session_close()

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
