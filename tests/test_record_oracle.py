"""The numpy restatement of the record write against records the reference's k_record_obs
wrote (tests/golden/record_state.npz, made by tests/golden/make_record_golden.py on a GPU box
from the reference's CUDA env), and its basic properties on synthetic states.  No GPU."""
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "record_state.npz")


def _state(z, tag):
    return {k[len(tag) + 1:]: z[k] for k in z.files if k.startswith(tag + "_") and k != tag + "_records"}


def test_record_oracle_reproduces_the_reference_records(oracle):
    z = np.load(GOLD)
    for tag in ("play", "fuzz"):
        st = _state(z, tag)
        assert set(st) == set(oracle.RECORD_FIELDS) | set(oracle.RECORD_MAPS)
        want = z[tag + "_records"]
        got = oracle.record_from_state(st)
        assert got.shape == want.shape == (32, 996)
        assert np.array_equal(got, want), tag
    # the fixture is not trivial: lit cells, items, mobs and non-zero scalars occur
    rec = z["fuzz_records"]
    cells = rec[:, :792].reshape(32, 99, 8)
    assert (cells[:, :, 2] == 1).any() and (cells[:, :, 1] > 1).any() and (cells[:, :, 3:] != 0).any()
    assert np.count_nonzero(rec[:, 792:].view(np.float32)) > 32 * 10


def test_record_oracle_properties_on_synthetic_state(oracle):
    st = oracle.synthetic_env_state(64, seed=3)
    rec = oracle.record_from_state(st)
    cells = rec[:, :792].reshape(64, 9, 11, 8)
    # an unlit or off-map cell carries no block, item or lit flag
    assert np.all((cells[..., 2] == 1) | ((cells[..., 0] == 0) & (cells[..., 1] == 0)))
    # the centre cell is the player's position: on the map, so lit iff light_map > 12 there
    env = np.arange(64)
    lvl, pr, pc = st["player_level"][0], st["player_position"][0], st["player_position"][1]
    assert np.array_equal(cells[:, 4, 5, 2] == 1, st["light_map"][env, lvl, pr, pc] > 12)
    # moving every mob out of the view removes the mob bytes and nothing else
    st2 = dict(st)
    st2["mob_position"] = st["mob_position"] + 100
    rec2 = oracle.record_from_state(st2)
    c2 = rec2[:, :792].reshape(64, 9, 11, 8)
    assert np.all(c2[..., 3:] == 0) and np.array_equal(c2[..., :3], cells[..., :3])
    assert np.array_equal(rec2[:, 792:], rec[:, 792:])
