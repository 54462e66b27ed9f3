"""Generates the committed fixtures under tests/golden/.

Run where the reference sources are present (they are compiled into
oracle/_ref/libcfref_env.so by oracle/Makefile):

    python tests/golden/make_golden.py

env_rollout_seed0.npz
    Records produced by the reference's own C environment (compact-obs build,
    craftax_full.c), 64 envs, seed 0, per-env xorshift action stream of its
    harness (craftax_full.c:8350-8353), auto-reset on; rows are the records
    seen BEFORE steps 200..211 together with the terminal flags of the step
    before each (what cu_rollout_step passes as prev_terminals).  Inputs of the
    path come from the reference itself, so they pin the record layout.
oracle_forward_seed0.npz
    What the CPU oracle computes on those records with a seeded N(0, 1/fan_in)
    arena (h256x2, 43 actions), free-running state from zero: per-step logits+value,
    sampled actions/logprobs for seeded uniforms, and the final state.  Guards the
    oracle against accidental change; it is not a reference output.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle as O  # noqa: E402

N, SEED, T0, T = 64, 0, 200, 12


def main():
    O.build()
    assert O.RefEnv.available(), "reference sources are needed to regenerate fixtures"
    env = O.RefEnv(N, SEED)
    recs, terms = [], []
    for t in range(T0 + T):
        if t >= T0:
            recs.append(env.records.copy())
            terms.append(env.terminals.copy())
        env.step_random()
    env.close()
    recs = np.stack(recs)
    terms = np.stack(terms)
    np.savez_compressed(os.path.join(HERE, "env_rollout_seed0.npz"), records=recs,
                        prev_terminals=terms, num_envs=N, seed=SEED, first_step=T0)
    print("records", recs.shape, "terminals set:", int(terms.sum()),
          "nonzero map bytes: %.3f" % (recs[..., :O.MAP] != 0).mean())

    H, L, A = 256, 2, 43
    params = O.init_weights(H, L, A, seed=7, scheme="normal")
    state = np.zeros((L, N, H), np.float32)
    rng = np.random.default_rng(11)
    u = rng.random((T, N), dtype=np.float32)
    lav, act, lp = [], [], []
    for t in range(T):
        l = O.forward(params, recs[t], terms[t], state, H, L, A)
        a, p = O.sample(l, u[t], A)
        lav.append(l), act.append(a), lp.append(p)
    np.savez_compressed(os.path.join(HERE, "oracle_forward_seed0.npz"), weight_seed=7,
                        uniforms=u, logits_av=np.stack(lav), actions=np.stack(act),
                        logprobs=np.stack(lp), final_state=state)
    print("oracle logits std %.3f" % np.stack(lav)[..., :A].std())


if __name__ == "__main__":
    main()
