/*
 * CPU oracle for the craftax.cu policy-rollout forward (TEST INFRASTRUCTURE).
 *
 * This file restates, in plain C, the arithmetic of the reference's batched
 * policy forward so that tests can check the CUDA path against it.  It is a
 * checker only: nothing in the shipped library links, loads or calls it.
 *
 * Parity status: the reference stores no golden vectors for this path (its
 * own gates are hashes of whole GPU rollouts, specific to one GPU
 * architecture and cuBLAS build).  The restatement is therefore pinned
 * procedurally: (1) records come from the reference's own C environment
 * compiled from its sources; (2) the expand and the sampler are integer /
 * single-op-exact and are compared bit for bit; (3) the forward follows the
 * reference's scalar fp32 policy kernel operation by operation.
 *
 * Layouts (reference craftax_full.cu:9086-9121):
 *   record   uint8[996]  = 792 map bytes + 51 raw little-endian fp32
 *   arena    W_enc[843][H] | b_enc[H] | W_gru[L][3H][H] | W_a[A][H] | b_a[A]
 *            | W_v[H] | b_v[1]                       (H = hidden, A = actions)
 *   state    float [L][n][H]  (layer-major, env-major, unit-minor;
 *            craftax_full.cu:9361,11984-12003)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CFXO_MAP 792
#define CFXO_TAIL 51
#define CFXO_OBS 843
#define CFXO_REC 996

/* Parameter-arena offsets, craftax_full.cu:9094-9102 with runtime H, L, A. */
typedef struct {
    size_t w_enc, b_enc, w_gru, w_a, b_a, w_v, b_v, count;
} cfxo_offsets;

static cfxo_offsets cfxo_layout(int H, int L, int A) {
    cfxo_offsets o;
    o.w_enc = 0;
    o.b_enc = (size_t)CFXO_OBS * H;
    o.w_gru = o.b_enc + H;
    o.w_a = o.w_gru + (size_t)L * 3 * H * H;
    o.b_a = o.w_a + (size_t)A * H;
    o.w_v = o.b_a + A;
    o.b_v = o.w_v + H;
    o.count = o.b_v + 1;
    return o;
}

size_t cfxo_param_count(int H, int L, int A) { return cfxo_layout(H, L, A).count; }

/*
 * Compact record -> 843 fp32 features.  Follows k_expand_obs
 * (craftax_full.cu:10028-10053): map bytes are converted with (float)byte,
 * the 51 tail floats are copied bit for bit.  out is [n][843].
 */
void cfxo_expand(const uint8_t* rec, float* out, int n) {
    for (int e = 0; e < n; e++) {
        const uint8_t* r = rec + (size_t)e * CFXO_REC;
        float* x = out + (size_t)e * CFXO_OBS;
        for (int f = 0; f < CFXO_MAP; f++) x[f] = (float)r[f];
        memcpy(x + CFXO_MAP, r + CFXO_MAP, CFXO_TAIL * sizeof(float));
    }
}

static float cfxo_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
/* cf_nn_mingru_g, craftax_full.cu:9136-9138 */
static float cfxo_g(float x) { return x >= 0.0f ? x + 0.5f : cfxo_sigmoid(x); }

/*
 * Categorical sample from logits with one uniform; follows
 * cf_nn_sample_action (craftax_full.cu:9147-9165) statement by statement:
 * running max, p[a] = expf(logit - m) summed in ascending a, first a with
 * u*total <= cumulative sum (default A-1), logprob = logit - m - logf(total).
 */
int cfxo_sample_one(const float* logits, int A, float u, float* logprob) {
    float m = logits[0];
    for (int a = 1; a < A; a++) m = fmaxf(m, logits[a]);
    float p[64];
    float total = 0.0f;
    for (int a = 0; a < A; a++) {
        p[a] = expf(logits[a] - m);
        total += p[a];
    }
    float target = u * total, cum = 0.0f;
    int action = A - 1;
    for (int a = 0; a < A; a++) {
        cum += p[a];
        if (target <= cum) { action = a; break; }
    }
    *logprob = logits[action] - m - logf(total);
    return action;
}

void cfxo_sample(const float* logits, int ld, int A, const float* u, int n,
                 int32_t* actions, float* logprobs) {
    for (int e = 0; e < n; e++)
        actions[e] = cfxo_sample_one(logits + (size_t)e * ld, A, u[e], &logprobs[e]);
}

/*
 * Scalar fp32 policy forward for n envs; follows k_policy_ref_l3
 * (craftax_full.cu:9778-9854) with runtime H, L, A:
 *   h = b_enc; for ascending feature f with x_f != 0: h[i] = fmaf(x_f, W_enc[f][i], h[i])
 *   per layer l, per unit k: three ascending-j fmaf dots zh, zg, zp over h;
 *     st = prev_terminal ? 0 : state;  out = st + sigmoid(zg)*(g(zh) - st);
 *     p = sigmoid(zp);  h2[k] = p*out + (1-p)*h[k];  state <- out
 *   logits[a] = b_a[a] + ascending fmaf dot;  value = b_v + ascending fmaf dot
 * Build with -ffp-contract=off: the reference compiles with -fmad=false
 * (Makefile:27), so only the explicit fmaf calls are fused.
 *
 * State layout here is the production one, [L][n][H] (k_mingru_epi_fwd,
 * craftax_full.cu:9361), not the scalar kernel's private [L][H][n].
 *
 * Outputs (any may be NULL): logits_av [n][A+1] with the value in column A
 * and biases INCLUDED (the production buffer holds them without biases,
 * craftax_full.cu:9725-9730; the difference is one fp32 add); h_last [n][H];
 * r_state [L][n][H] = the post-zero state inputs (craftax_full.cu:9369-9375).
 */
void cfxo_forward(const float* params, int H, int L, int A,
                  const uint8_t* rec, const float* prev_terminals,
                  float* state, int n,
                  float* logits_av, float* h_last, float* r_state) {
    cfxo_offsets o = cfxo_layout(H, L, A);
    const float* W_enc = params + o.w_enc;
    const float* b_enc = params + o.b_enc;
    const float* W_gru = params + o.w_gru;
    const float* W_a = params + o.w_a;
    const float* b_a = params + o.b_a;
    const float* W_v = params + o.w_v;
    const float* b_v = params + o.b_v;
#pragma omp parallel
    {
        float* h = (float*)malloc(sizeof(float) * H);
        float* h2 = (float*)malloc(sizeof(float) * H);
#pragma omp for schedule(static)
        for (int e = 0; e < n; e++) {
            const uint8_t* r = rec + (size_t)e * CFXO_REC;
            for (int i = 0; i < H; i++) h[i] = b_enc[i];
            for (int f = 0; f < CFXO_OBS; f++) {
                float xf;
                if (f < CFXO_MAP) xf = (float)r[f];
                else memcpy(&xf, r + CFXO_MAP + 4 * (f - CFXO_MAP), 4);
                if (xf == 0.0f) continue;
                const float* col = W_enc + (size_t)f * H;
                for (int i = 0; i < H; i++) h[i] = fmaf(xf, col[i], h[i]);
            }
            int dz = prev_terminals != NULL && prev_terminals[e] != 0.0f;
            for (int l = 0; l < L; l++) {
                const float* Wl = W_gru + (size_t)l * 3 * H * H;
                float* st_row = state + ((size_t)l * n + e) * H;
                for (int k = 0; k < H; k++) {
                    float st = dz ? 0.0f : st_row[k];
                    if (r_state) r_state[((size_t)l * n + e) * H + k] = st;
                    float zh = 0.0f, zg = 0.0f, zp = 0.0f;
                    const float* wh = Wl + (size_t)k * H;
                    const float* wg = Wl + (size_t)(H + k) * H;
                    const float* wp = Wl + (size_t)(2 * H + k) * H;
                    for (int j = 0; j < H; j++) {
                        zh = fmaf(wh[j], h[j], zh);
                        zg = fmaf(wg[j], h[j], zg);
                        zp = fmaf(wp[j], h[j], zp);
                    }
                    float out = st + cfxo_sigmoid(zg) * (cfxo_g(zh) - st);
                    float p = cfxo_sigmoid(zp);
                    h2[k] = p * out + (1.0f - p) * h[k];
                    st_row[k] = out;
                }
                memcpy(h, h2, sizeof(float) * H);
            }
            if (h_last) memcpy(h_last + (size_t)e * H, h, sizeof(float) * H);
            if (logits_av) {
                float* lo = logits_av + (size_t)e * (A + 1);
                for (int a = 0; a < A; a++) {
                    float z = b_a[a];
                    const float* wa = W_a + (size_t)a * H;
                    for (int j = 0; j < H; j++) z = fmaf(wa[j], h[j], z);
                    lo[a] = z;
                }
                float v = b_v[0];
                for (int j = 0; j < H; j++) v = fmaf(W_v[j], h[j], v);
                lo[A] = v;
            }
        }
        free(h);
        free(h2);
    }
}

/* ------------------------------------------------------------------------------------
 * Classic game (reference craftax_classic.cu).  Record: uint8[148] = 63 block ids (int8,
 * 0..16), 63 mob bit masks (1 zombie, 2 cow, 4 skeleton, 8 arrow), 12 inventory counts and
 * health, food, drink, energy (int8, 0..9), direction (1..4), sleeping flag, light level as
 * raw fp32 (craftax_classic.cu:50-59, writer :1574-1604).  Features: 63 cells x (17 block
 * one-hot + 4 mob bits) = 1323, then inventory/10 x12, intrinsics/10 x4, direction one-hot
 * x4, light, sleeping = 1345 (expand_obs_kernel :1265-1301).  Arena: same order as the full
 * game with 1345 encoder rows (:1526-1533).  Policy: 3 MinGRU layers, 17 actions.
 * ------------------------------------------------------------------------------------ */
#define CFXO_C_CELLS 63
#define CFXO_C_BLOCKS 17
#define CFXO_C_INV 12
#define CFXO_C_OBS 1345
#define CFXO_C_REC 148

size_t cfxo_classic_param_count(int H, int L, int A) {
    return (size_t)CFXO_C_OBS * H + H + (size_t)L * 3 * H * H + (size_t)A * H + A + H + 1;
}

/* expand_obs_kernel (:1265-1301): out is [n][1345]. */
void cfxo_classic_expand(const uint8_t* rec, float* out, int n) {
    for (int e = 0; e < n; e++) {
        const uint8_t* c = rec + (size_t)e * CFXO_C_REC;
        float* o = out + (size_t)e * CFXO_C_OBS;
        int k = 0;
        for (int cell = 0; cell < CFXO_C_CELLS; cell++) {
            int8_t blk = (int8_t)c[cell];
            for (int b = 0; b < CFXO_C_BLOCKS; b++) o[k++] = (blk == b) ? 1.0f : 0.0f;
            uint8_t m = c[CFXO_C_CELLS + cell];
            for (int j = 0; j < 4; j++) o[k++] = (m & (1 << j)) ? 1.0f : 0.0f;
        }
        int i2 = 2 * CFXO_C_CELLS;
        for (int j = 0; j < CFXO_C_INV + 4; j++) o[k++] = (float)(int8_t)c[i2++] / 10.0f;
        int8_t dir = (int8_t)c[i2++];
        for (int d = 1; d <= 4; d++) o[k++] = (dir == d) ? 1.0f : 0.0f;
        uint8_t sleeping = c[i2++];
        float light;
        memcpy(&light, c + i2, 4);
        o[k++] = light;
        o[k++] = sleeping ? 1.0f : 0.0f;
    }
}

/* Forward in the order of encode_obs_kernel (:1714-1751) for the encoder - bias first, then
 * per cell the block column and the set mob bits, then the 22 scalar features, every term
 * as fmaf(x, W, acc) - and of ref_policy_l3_kernel (:2016-2047) for the layers and the heads
 * (logits = b_a + dot, value = b_v + dot).  prev_done: int8 flags or NULL.  State [L][n][H]. */
void cfxo_classic_forward(const float* params, int H, int L, int A,
                          const uint8_t* rec, const int8_t* prev_done,
                          float* state, int n, float* logits_av, float* h_enc_out) {
    const float* W_enc = params;
    const float* b_enc = W_enc + (size_t)CFXO_C_OBS * H;
    const float* W_gru = b_enc + H;
    const float* W_a = W_gru + (size_t)L * 3 * H * H;
    const float* b_a = W_a + (size_t)A * H;
    const float* W_v = b_a + A;
    const float* b_v = W_v + H;
#pragma omp parallel
    {
        float* h = (float*)malloc(sizeof(float) * H);
        float* h2 = (float*)malloc(sizeof(float) * H);
#pragma omp for schedule(static)
        for (int e = 0; e < n; e++) {
            const uint8_t* c = rec + (size_t)e * CFXO_C_REC;
            for (int i = 0; i < H; i++) h[i] = b_enc[i];
            for (int cell = 0; cell < CFXO_C_CELLS; cell++) {
                const float* col = W_enc + (size_t)(cell * (CFXO_C_BLOCKS + 4) + (int8_t)c[cell]) * H;
                for (int i = 0; i < H; i++) h[i] = fmaf(1.0f, col[i], h[i]);
                uint8_t m = c[CFXO_C_CELLS + cell];
                int fm = cell * (CFXO_C_BLOCKS + 4) + CFXO_C_BLOCKS;
                for (int j = 0; j < 4; j++)
                    if (m & (1 << j)) {
                        const float* mc = W_enc + (size_t)(fm + j) * H;
                        for (int i = 0; i < H; i++) h[i] = fmaf(1.0f, mc[i], h[i]);
                    }
            }
            int oi = 2 * CFXO_C_CELLS, f = CFXO_C_CELLS * (CFXO_C_BLOCKS + 4);
            for (int j = 0; j < CFXO_C_INV + 4; j++, f++) {
                float x = (float)(int8_t)c[oi++] / 10.0f;
                const float* col = W_enc + (size_t)f * H;
                for (int i = 0; i < H; i++) h[i] = fmaf(x, col[i], h[i]);
            }
            int8_t dir = (int8_t)c[oi++];
            for (int d = 1; d <= 4; d++, f++) {
                float x = (dir == d) ? 1.0f : 0.0f;
                const float* col = W_enc + (size_t)f * H;
                for (int i = 0; i < H; i++) h[i] = fmaf(x, col[i], h[i]);
            }
            uint8_t sleeping = c[oi++];
            float light;
            memcpy(&light, c + oi, 4);
            {
                const float* col = W_enc + (size_t)f * H; f++;
                for (int i = 0; i < H; i++) h[i] = fmaf(light, col[i], h[i]);
                col = W_enc + (size_t)f * H;
                float x = sleeping ? 1.0f : 0.0f;
                for (int i = 0; i < H; i++) h[i] = fmaf(x, col[i], h[i]);
            }
            if (h_enc_out) memcpy(h_enc_out + (size_t)e * H, h, sizeof(float) * H);
            int dz = prev_done != NULL && prev_done[e] != 0;
            for (int l = 0; l < L; l++) {
                const float* Wl = W_gru + (size_t)l * 3 * H * H;
                float* st_row = state + ((size_t)l * n + e) * H;
                for (int k = 0; k < H; k++) {
                    float st = dz ? 0.0f : st_row[k];
                    float zh = 0.0f, zg = 0.0f, zp = 0.0f;
                    const float* wh = Wl + (size_t)k * H;
                    const float* wg = Wl + (size_t)(H + k) * H;
                    const float* wp = Wl + (size_t)(2 * H + k) * H;
                    for (int j = 0; j < H; j++) {
                        zh = fmaf(wh[j], h[j], zh);
                        zg = fmaf(wg[j], h[j], zg);
                        zp = fmaf(wp[j], h[j], zp);
                    }
                    float out = st + cfxo_sigmoid(zg) * (cfxo_g(zh) - st);
                    float p = cfxo_sigmoid(zp);
                    h2[k] = p * out + (1.0f - p) * h[k];
                    st_row[k] = out;
                }
                memcpy(h, h2, sizeof(float) * H);
            }
            if (logits_av) {
                float* lo = logits_av + (size_t)e * (A + 1);
                for (int a = 0; a < A; a++) {
                    float z = b_a[a];
                    const float* wa = W_a + (size_t)a * H;
                    for (int j = 0; j < H; j++) z = fmaf(wa[j], h[j], z);
                    lo[a] = z;
                }
                float v = b_v[0];
                for (int j = 0; j < H; j++) v = fmaf(W_v[j], h[j], v);
                lo[A] = v;
            }
        }
        free(h);
        free(h2);
    }
}

int cfxo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void cfxo_set_threads(int t) {
#ifdef _OPENMP
    if (t > 0) omp_set_num_threads(t);
#else
    (void)t;
#endif
}
