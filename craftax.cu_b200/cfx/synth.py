"""Seeded synthetic inputs of the policy forward: parameter arenas and compact
observation records with the value ranges of real Craftax records.  Used by the
benchmark and the tests; stands in for environment trajectories."""
import numpy as np

MAP, TAIL, OBS, REC = 792, 51, 843, 996


def offsets(H=256, L=2, A=43):
    """Arena offsets in reference order (craftax_full.cu:9094-9102)."""
    o = {}
    o["w_enc"] = 0
    o["b_enc"] = OBS * H
    o["w_gru"] = o["b_enc"] + H
    o["w_a"] = o["w_gru"] + L * 3 * H * H
    o["b_a"] = o["w_a"] + A * H
    o["w_v"] = o["b_a"] + A
    o["b_v"] = o["w_v"] + H
    o["count"] = o["b_v"] + 1
    return o


def init_weights(H=256, L=2, A=43, seed=0, scheme="normal"):
    """Seeded parameter arena.

    scheme "normal":  weights N(0, 1/fan_in), biases zero (benchmark configs).
    scheme "uniform": weights and biases U(+-1/sqrt(fan_in)), the distribution
    of the reference's own initialiser (craftax_full.cu:11830-11845)."""
    o = offsets(H, L, A)
    rng = np.random.default_rng(seed)
    p = np.zeros(o["count"], np.float32)
    segs = [("w_enc", OBS * H, OBS, False), ("b_enc", H, OBS, True),
            ("w_gru", L * 3 * H * H, H, False), ("w_a", A * H, H, False),
            ("b_a", A, H, True), ("w_v", H, H, False), ("b_v", 1, H, True)]
    for name, cnt, fan, is_bias in segs:
        if scheme == "normal":
            v = np.zeros(cnt) if is_bias else rng.normal(0.0, 1.0 / np.sqrt(fan), cnt)
        else:
            b = 1.0 / np.sqrt(fan)
            v = rng.uniform(-b, b, cnt)
        p[o[name]:o[name] + cnt] = v.astype(np.float32)
    return p


def synthetic_records(n, seed=4):
    """Seeded synthetic records: every map byte uniform over its channel's valid
    range, tail floats drawn from their quantised value sets
    (ranges: craftax_full.c:573-577, 2646-2703)."""
    rng = np.random.default_rng(seed)
    rec = np.zeros((n, REC), np.uint8)
    hi = np.array([37, 6, 2, 9, 9, 9, 9, 9])
    m = rng.integers(0, np.tile(hi, 99)[None, :], size=(n, MAP))
    rec[:, :MAP] = m.astype(np.uint8)
    t = np.zeros((n, TAIL), np.float32)
    k = rng.integers(0, 100, size=(n, 10)).astype(np.float32)
    t[:, 0:10] = np.sqrt(k) * np.float32(0.1)
    t[:, 10] = rng.integers(0, 3, n) * np.float32(0.5)
    t[:, 11] = rng.integers(0, 5, n) * np.float32(0.25)
    t[:, 12] = rng.integers(0, 5, n) * np.float32(0.25)
    t[:, 13:16] = rng.integers(0, 2, (n, 3))
    k = rng.integers(0, 100, size=(n, 6)).astype(np.float32)
    t[:, 16:22] = np.sqrt(k) * np.float32(0.1)
    t[:, 22:31] = rng.integers(0, 10, (n, 9)).astype(np.float32) * np.float32(0.1)
    d = rng.integers(0, 4, n)
    t[np.arange(n), 31 + d] = 1.0
    t[:, 35:39] = rng.integers(0, 3, (n, 4)) * np.float32(0.5)
    t[:, 39:43] = rng.integers(0, 3, (n, 4))
    t[:, 43] = rng.random(n, dtype=np.float32)
    t[:, 44:48] = rng.integers(0, 2, (n, 4))
    t[:, 48] = rng.integers(0, 9, n) * np.float32(0.1)
    t[:, 49:51] = rng.integers(0, 2, (n, 2))
    rec[:, MAP:] = t.view(np.uint8).reshape(n, TAIL * 4)
    return rec


# ---- classic game (148-byte records, 1345 features; reference craftax_classic.cu:38-59) ----
CLASSIC_OBS, CLASSIC_REC, CLASSIC_CELLS = 1345, 148, 63


def classic_offsets(H, L, A):
    o = {"w_enc": 0, "b_enc": CLASSIC_OBS * H}
    o["w_gru"] = o["b_enc"] + H
    o["w_a"] = o["w_gru"] + L * 3 * H * H
    o["b_a"] = o["w_a"] + A * H
    o["w_v"] = o["b_a"] + A
    o["b_v"] = o["w_v"] + H
    o["count"] = o["b_v"] + 1
    return o


def classic_init_weights(H=256, L=3, A=17, seed=0):
    """N(0, 1/fan_in) weights; biases drawn too (small) so that every arena segment matters."""
    rng = np.random.default_rng(seed)
    o = classic_offsets(H, L, A)
    p = np.empty(o["count"], np.float32)
    p[:o["b_enc"]] = rng.normal(0, 1 / np.sqrt(85.0), CLASSIC_OBS * H)     # ~85 active features per record
    p[o["b_enc"]:o["w_gru"]] = rng.normal(0, 0.05, H)
    p[o["w_gru"]:o["w_a"]] = rng.normal(0, 1 / np.sqrt(H), L * 3 * H * H)
    p[o["w_a"]:o["b_a"]] = rng.normal(0, 1 / np.sqrt(H), A * H)
    p[o["b_a"]:o["w_v"]] = rng.normal(0, 0.05, A)
    p[o["w_v"]:o["b_v"]] = rng.normal(0, 1 / np.sqrt(H), H)
    p[o["b_v"]] = 0.1
    return p


def classic_synthetic_records(n, seed=0):
    """Seeded records over the valid ranges of the classic layout: block ids 0..16, mob masks
    with each of the four bits set with probability 0.05, inventory and intrinsics 0..9,
    direction 1..4, sleeping 0/1, light in [0, 1] as raw fp32."""
    rng = np.random.default_rng(seed)
    rec = np.zeros((n, CLASSIC_REC), np.uint8)
    rec[:, :63] = rng.integers(0, 17, (n, 63))
    rec[:, 63:126] = (rng.random((n, 63, 4)) < 0.05).astype(np.uint8) @ np.array([1, 2, 4, 8], np.uint8)
    rec[:, 126:142] = rng.integers(0, 10, (n, 16))
    rec[:, 142] = rng.integers(1, 5, n)
    rec[:, 143] = rng.integers(0, 2, n)
    rec[:, 144:148] = rng.random(n, dtype=np.float32).reshape(n, 1).view(np.uint8)
    return rec
