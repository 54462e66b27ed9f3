/*
 * The reference's classic-game policy kernels behind a C ABI (TEST INFRASTRUCTURE; compiled
 * only where the reference sources are present, into oracle/_ref/, never committed).
 *
 * craftax_classic.cu is the reference's kernel translation unit (main_classic.cu includes
 * it).  This file includes it the same way (path given with -DCFX_REF_CLASSIC_CU) and runs
 * its UNMODIFIED kernels on caller-provided records, weights and state:
 *   expand_obs_kernel (:1265), encode_obs_kernel (:1714), mingru_epi_fwd_kernel (:1761),
 *   value_sample_kernel (:1841), with the gate and logit products done by cublasSgemm in
 *   default (fp32) math exactly where Rollout::step (main_classic.cu:439-474) calls cuBLAS.
 * Built with the reference Makefile's classic flags (--use_fast_math).
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cublas_v2.h>
#include CFX_REF_CLASSIC_CU

#define RC_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)
#define RC_BLAS(x) do { cublasStatus_t s_ = (x); if (s_ != CUBLAS_STATUS_SUCCESS) { \
    fprintf(stderr, "cuBLAS error %d at %s:%d\n", (int)s_, __FILE__, __LINE__); exit(1); } } while (0)

extern "C" {

int refcl_hidden(void) { return HIDDEN; }
int refcl_layers(void) { return GRU_LAYERS; }
int refcl_actions(void) { return NUM_ACTIONS; }
int refcl_obs(void) { return OBS_DIM; }
int refcl_record_bytes(void) { return OBS_DIM_COMPACT; }
int refcl_param_count(void) { return PARAM_COUNT; }

/* device pointers in and out */
void refcl_expand(const uint8_t* d_rec, float* d_out, int n) {
    expand_obs_kernel<<<(n + 127) / 128, 128>>>(d_rec, d_out, n);
    RC_CHECK(cudaGetLastError());
    RC_CHECK(cudaDeviceSynchronize());
}

/* One forward of the batched pipeline.  d_params: arena (:1526-1533); d_state: [L][n][H],
 * updated in place; d_prev_done: int8 [n] or NULL.  Host outputs: logits_av [n][A+1] (biases
 * added, value in column A), h_enc [n][H], actions, logprobs. */
void refcl_forward(const float* d_params, const uint8_t* d_rec, const int8_t* d_prev_done,
                   float* d_state, int n, unsigned long long seed, unsigned long long step,
                   float* logits_av, float* h_enc_out, int* actions, float* logprobs) {
    static cublasHandle_t blas = NULL;
    if (!blas) {
        RC_BLAS(cublasCreate(&blas));
        RC_BLAS(cublasSetMathMode(blas, CUBLAS_DEFAULT_MATH));
    }
    const float* W_enc = d_params + PARAM_W_ENC;
    const float* b_enc = d_params + PARAM_B_ENC;
    const float* W_gru = d_params + PARAM_W_GRU;
    const float* W_a = d_params + PARAM_W_A;
    const float* b_a = d_params + PARAM_B_A;
    const float* W_v = d_params + PARAM_W_V;
    const float* b_v = d_params + PARAM_B_V;
    const size_t hn = (size_t)HIDDEN * n;
    float *h0, *h1, *pre, *logits, *d_lp, *d_val;
    int32_t* d_act;
    uint64_t* d_ctr;
    RC_CHECK(cudaMalloc(&h0, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&h1, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&pre, (size_t)GRU_OUT * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&logits, (size_t)NUM_ACTIONS * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_lp, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_val, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_act, (size_t)n * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&d_ctr, sizeof(uint64_t)));
    uint64_t ctr = step;
    RC_CHECK(cudaMemcpy(d_ctr, &ctr, sizeof(ctr), cudaMemcpyHostToDevice));
    RC_CHECK(cudaDeviceSynchronize());
    RC_BLAS(cublasSetStream(blas, 0));

    encode_obs_kernel<<<(int)((hn + 255) / 256), 256>>>(d_rec, W_enc, b_enc, h0, 0, n, n, n, 0);
    RC_CHECK(cudaGetLastError());
    if (h_enc_out) RC_CHECK(cudaMemcpy(h_enc_out, h0, hn * sizeof(float), cudaMemcpyDeviceToHost));
    const float one = 1.0f, zero = 0.0f;
    float* x = h0;
    float* y = h1;
    for (int l = 0; l < GRU_LAYERS; l++) {
        RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, GRU_OUT, n, HIDDEN, &one,
                            W_gru + (size_t)l * GRU_OUT * HIDDEN, HIDDEN, x, HIDDEN, &zero, pre, GRU_OUT));
        mingru_epi_fwd_kernel<<<(int)((hn + 255) / 256), 256>>>(pre, x, d_state + (size_t)l * hn, y, NULL,
                                                                d_prev_done, n);
        RC_CHECK(cudaGetLastError());
        float* t = x; x = y; y = t;
    }
    RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, NUM_ACTIONS, n, HIDDEN, &one, W_a, HIDDEN, x, HIDDEN,
                        &zero, logits, NUM_ACTIONS));
    value_sample_kernel<<<(n + 255) / 256, 256>>>(x, logits, b_a, W_v, b_v, d_act, d_lp, d_val, n, seed, d_ctr);
    RC_CHECK(cudaGetLastError());
    RC_CHECK(cudaDeviceSynchronize());

    float* hl = (float*)malloc((size_t)NUM_ACTIONS * n * sizeof(float));
    float* hv = (float*)malloc((size_t)n * sizeof(float));
    float hb[NUM_ACTIONS];
    RC_CHECK(cudaMemcpy(hl, logits, (size_t)NUM_ACTIONS * n * sizeof(float), cudaMemcpyDeviceToHost));
    RC_CHECK(cudaMemcpy(hv, d_val, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    RC_CHECK(cudaMemcpy(hb, b_a, sizeof(hb), cudaMemcpyDeviceToHost));
    for (int e = 0; e < n; e++) {
        for (int a = 0; a < NUM_ACTIONS; a++)
            logits_av[(size_t)e * (NUM_ACTIONS + 1) + a] = hl[(size_t)e * NUM_ACTIONS + a] + hb[a];
        logits_av[(size_t)e * (NUM_ACTIONS + 1) + NUM_ACTIONS] = hv[e];
    }
    if (actions) RC_CHECK(cudaMemcpy(actions, d_act, (size_t)n * sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (logprobs) RC_CHECK(cudaMemcpy(logprobs, d_lp, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    free(hl); free(hv);
    cudaFree(h0); cudaFree(h1); cudaFree(pre); cudaFree(logits); cudaFree(d_lp); cudaFree(d_val);
    cudaFree(d_act); cudaFree(d_ctr);
}

/* Times the record-driven forward (encode_obs_kernel, three Sgemm + mingru_epi_fwd_kernel,
 * logits Sgemm, value_sample_kernel, bump) on device-resident inputs: `warm` untimed and `iters`
 * timed repetitions, CUDA events on the default stream.  tf32 != 0 selects the math mode the
 * reference's rollout uses (CUBLAS_TF32_TENSOR_OP_MATH, main_classic.cu:283).  Returns ms per
 * forward. */
float refcl_time_forward(const float* d_params, const uint8_t* d_rec, const int8_t* d_prev_done,
                         float* d_state, int n, int warm, int iters, int tf32) {
    cublasHandle_t blas;
    RC_BLAS(cublasCreate(&blas));
    RC_BLAS(cublasSetMathMode(blas, tf32 ? CUBLAS_TF32_TENSOR_OP_MATH : CUBLAS_DEFAULT_MATH));
    const float* W_enc = d_params + PARAM_W_ENC;
    const float* b_enc = d_params + PARAM_B_ENC;
    const float* W_gru = d_params + PARAM_W_GRU;
    const float* W_a = d_params + PARAM_W_A;
    const float* b_a = d_params + PARAM_B_A;
    const float* W_v = d_params + PARAM_W_V;
    const float* b_v = d_params + PARAM_B_V;
    const size_t hn = (size_t)HIDDEN * n;
    float *h0, *h1, *pre, *logits, *d_lp, *d_val;
    int32_t* d_act;
    uint64_t* d_ctr;
    RC_CHECK(cudaMalloc(&h0, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&h1, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&pre, (size_t)GRU_OUT * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&logits, (size_t)NUM_ACTIONS * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_lp, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_val, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_act, (size_t)n * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&d_ctr, sizeof(uint64_t)));
    RC_CHECK(cudaMemset(d_ctr, 0, sizeof(uint64_t)));
    RC_BLAS(cublasSetStream(blas, 0));
    const float one = 1.0f, zero = 0.0f;
    cudaEvent_t ea, eb;
    RC_CHECK(cudaEventCreate(&ea));
    RC_CHECK(cudaEventCreate(&eb));
    for (int it = 0; it < warm + iters; it++) {
        if (it == warm) RC_CHECK(cudaEventRecord(ea, 0));
        encode_obs_kernel<<<(int)((hn + 255) / 256), 256>>>(d_rec, W_enc, b_enc, h0, 0, n, n, n, 0);
        float* x = h0;
        float* y = h1;
        for (int l = 0; l < GRU_LAYERS; l++) {
            RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, GRU_OUT, n, HIDDEN, &one,
                                W_gru + (size_t)l * GRU_OUT * HIDDEN, HIDDEN, x, HIDDEN, &zero, pre, GRU_OUT));
            mingru_epi_fwd_kernel<<<(int)((hn + 255) / 256), 256>>>(pre, x, d_state + (size_t)l * hn, y, NULL,
                                                                    d_prev_done, n);
            float* t = x; x = y; y = t;
        }
        RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, NUM_ACTIONS, n, HIDDEN, &one, W_a, HIDDEN, x, HIDDEN,
                            &zero, logits, NUM_ACTIONS));
        value_sample_kernel<<<(n + 255) / 256, 256>>>(x, logits, b_a, W_v, b_v, d_act, d_lp, d_val, n, 1, d_ctr);
        bump_ctr_kernel<<<1, 1>>>(d_ctr);
    }
    RC_CHECK(cudaEventRecord(eb, 0));
    RC_CHECK(cudaGetLastError());
    RC_CHECK(cudaDeviceSynchronize());
    float ms = 0.f;
    RC_CHECK(cudaEventElapsedTime(&ms, ea, eb));
    cudaEventDestroy(ea); cudaEventDestroy(eb);
    cudaFree(h0); cudaFree(h1); cudaFree(pre); cudaFree(logits); cudaFree(d_lp); cudaFree(d_val);
    cudaFree(d_act); cudaFree(d_ctr);
    cublasDestroy(blas);
    return ms / (float)iters;
}

#ifdef CFX_REF_WITH_CFX
#include "cfx.h"
/* ---- lock-step classic rollout: the reference's classic env kernels (reset_all_warp_kernel
 * :1443, record_obs_kernel :1884, step_mark_kernel :1401, reset_warp_ctr_kernel :1908,
 * bump_ctr_kernel :1929, in the order of Rollout::step, main_classic.cu:439-474), driven by
 * this library's classic forward, with the reference's record-driven classic pipeline
 * (encode_obs_kernel, cublasSgemm + mingru_epi_fwd_kernel per layer, logits Sgemm,
 * value_sample_kernel) consuming the same 148-byte records beside it.  Both keep their own
 * recurrent state, zeroed from the previous step's dones and never at t = 0
 * (main_classic.cu:436-443).  tf32 != 0 runs the reference products in the math mode its
 * rollout uses (main_classic.cu:283) instead of strict fp32.  The comparison runs on the device
 * every step.  out[0] max |dlogit|, out[1] max |dvalue|, out[2] fraction of env-steps with the
 * same greedy action, out[3] with the same sampled action (same Philox draw), out[4] episode
 * ends seen, out[5] max |logit|, out[6] env-steps compared.  Returns 0, or 1 when a cfx call
 * failed (message on stderr). */
__global__ void refcl_k_compare(const float* __restrict__ ref_logits, const float* __restrict__ b_a,
                                const float* __restrict__ ref_val, const float* __restrict__ cfx_lav,
                                const int32_t* __restrict__ ref_act, const int32_t* __restrict__ cfx_act,
                                int n, unsigned* fmax, unsigned long long* counts) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const float* r = ref_logits + (size_t)e * NUM_ACTIONS;
    const float* c = cfx_lav + (size_t)e * (NUM_ACTIONS + 1);
    float dmax = 0.f, lmax = 0.f, rbest = 0.f, cbest = 0.f;
    int ra = 0, ca = 0;
    for (int a = 0; a < NUM_ACTIONS; a++) {
        const float rl = r[a] + b_a[a], cl = c[a];
        dmax = fmaxf(dmax, fabsf(rl - cl));
        lmax = fmaxf(lmax, fabsf(rl));
        if (a == 0 || rl > rbest) { rbest = rl; ra = a; }
        if (a == 0 || cl > cbest) { cbest = cl; ca = a; }
    }
    atomicMax(&fmax[0], __float_as_uint(dmax));   /* non-negative floats order like their bits */
    atomicMax(&fmax[1], __float_as_uint(fabsf(ref_val[e] - c[NUM_ACTIONS])));
    atomicMax(&fmax[2], __float_as_uint(lmax));
    if (ra == ca) atomicAdd(&counts[0], 1ULL);
    if (ref_act[e] == cfx_act[e]) atomicAdd(&counts[1], 1ULL);
}

__global__ void refcl_k_count_done(const int8_t* __restrict__ done, int n, unsigned long long* counts) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n && done[e]) atomicAdd(&counts[2], 1ULL);
}

int refcl_lockstep(int n, int steps, unsigned long long seed, const float* host_params, int precision,
                   int tf32, double* out) {
    cublasHandle_t blas;
    RC_BLAS(cublasCreate(&blas));
    RC_BLAS(cublasSetMathMode(blas, tf32 ? CUBLAS_TF32_TENSOR_OP_MATH : CUBLAS_DEFAULT_MATH));
    cudaStream_t st;
    RC_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    RC_BLAS(cublasSetStream(blas, st));
    uint8_t* arena;
    RC_CHECK(cudaMalloc(&arena, soa_bytes(n)));
    RC_CHECK(cudaMemset(arena, 0, soa_bytes(n)));
    EnvSoA g = carve_soa(arena, n);
    float* d_params;
    RC_CHECK(cudaMalloc(&d_params, (size_t)PARAM_COUNT * sizeof(float)));
    RC_CHECK(cudaMemcpy(d_params, host_params, (size_t)PARAM_COUNT * sizeof(float), cudaMemcpyHostToDevice));
    const float* W_enc = d_params + PARAM_W_ENC;
    const float* b_enc = d_params + PARAM_B_ENC;
    const float* W_gru = d_params + PARAM_W_GRU;
    const float* W_a = d_params + PARAM_W_A;
    const float* b_a = d_params + PARAM_B_A;
    const float* W_v = d_params + PARAM_W_V;
    const float* b_v = d_params + PARAM_B_V;
    const size_t hn = (size_t)HIDDEN * n;
    float *h0, *h1, *pre, *logits, *ref_state, *ref_lp, *ref_val, *rewards, *term, *d_lav;
    int32_t *ref_act, *cfx_act, *reset_list, *reset_ctrl;
    int8_t* done[2];
    uint8_t* rec;
    uint64_t* step_ctr;
    unsigned* d_fmax;
    unsigned long long* d_counts;
    RC_CHECK(cudaMalloc(&h0, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&h1, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&pre, (size_t)GRU_OUT * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&logits, (size_t)NUM_ACTIONS * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&ref_state, (size_t)GRU_LAYERS * hn * sizeof(float)));
    RC_CHECK(cudaMemset(ref_state, 0, (size_t)GRU_LAYERS * hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&ref_lp, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&ref_val, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&rewards, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&term, (size_t)n * sizeof(float)));
    RC_CHECK(cudaMalloc(&d_lav, (size_t)n * (NUM_ACTIONS + 1) * sizeof(float)));
    RC_CHECK(cudaMalloc(&ref_act, (size_t)n * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&cfx_act, (size_t)n * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&reset_list, (size_t)n * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&reset_ctrl, 2 * sizeof(int32_t)));
    RC_CHECK(cudaMalloc(&done[0], (size_t)n));
    RC_CHECK(cudaMalloc(&done[1], (size_t)n));
    RC_CHECK(cudaMalloc(&rec, (size_t)n * OBS_DIM_COMPACT));
    RC_CHECK(cudaMalloc(&step_ctr, sizeof(uint64_t)));
    RC_CHECK(cudaMemset(step_ctr, 0, sizeof(uint64_t)));
    RC_CHECK(cudaMalloc(&d_fmax, 4 * sizeof(unsigned)));
    RC_CHECK(cudaMalloc(&d_counts, 4 * sizeof(unsigned long long)));
    RC_CHECK(cudaMemset(d_fmax, 0, 4 * sizeof(unsigned)));
    RC_CHECK(cudaMemset(d_counts, 0, 4 * sizeof(unsigned long long)));
    int dev = 0, rc = 0;
    RC_CHECK(cudaGetDevice(&dev));
    cfx_policy* cp = NULL;
    if (cfx_policy_create_classic(&cp, dev, n, HIDDEN, GRU_LAYERS, NUM_ACTIONS, precision) != CFX_OK ||
        cfx_policy_set_weights(cp, d_params, PARAM_COUNT, 1) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        rc = 1;
    }
    const int block = 256, grid = (n + block - 1) / block;
    {
        int wgrid = (int)(((size_t)n * 32 + RESET_WARP_BLOCK - 1) / RESET_WARP_BLOCK);
        reset_all_warp_kernel<<<wgrid, RESET_WARP_BLOCK, 0, st>>>(g, n, seed);
        RC_CHECK(cudaGetLastError());
        RC_CHECK(cudaStreamSynchronize(st));
    }
    const float one = 1.0f, zero = 0.0f;
    for (int t = 0; t < steps && rc == 0; t++) {
        const int8_t* prev = (t == 0) ? NULL : done[(t - 1) & 1];
        RC_CHECK(cudaMemsetAsync(reset_ctrl, 0, 8, st));
        record_obs_kernel<<<grid, block, 0, st>>>(g, rec, n);
        /* reference pipeline on the records */
        encode_obs_kernel<<<(int)((hn + 255) / 256), 256, 0, st>>>(rec, W_enc, b_enc, h0, 0, n, n, n, 0);
        float* x = h0;
        float* y = h1;
        for (int l = 0; l < GRU_LAYERS; l++) {
            RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, GRU_OUT, n, HIDDEN, &one,
                                W_gru + (size_t)l * GRU_OUT * HIDDEN, HIDDEN, x, HIDDEN, &zero, pre, GRU_OUT));
            mingru_epi_fwd_kernel<<<(int)((hn + 255) / 256), 256, 0, st>>>(pre, x, ref_state + (size_t)l * hn, y,
                                                                           NULL, prev, n);
            float* tmp = x; x = y; y = tmp;
        }
        RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, NUM_ACTIONS, n, HIDDEN, &one, W_a, HIDDEN, x, HIDDEN,
                            &zero, logits, NUM_ACTIONS));
        value_sample_kernel<<<grid, block, 0, st>>>(x, logits, b_a, W_v, b_v, ref_act, ref_lp, ref_val, n, seed,
                                                    step_ctr);
        /* path under test */
        if (prev && cfx_classic_done_to_terminals(dev, prev, term, n, st) != CFX_OK) rc = 1;
        cfx_forward_io io;
        memset(&io, 0, sizeof(io));
        io.records = rec;
        io.prev_terminals = prev ? term : NULL;
        io.actions = cfx_act;
        io.logits_av = d_lav;
        io.seed = seed;
        io.bump_step = 1;
        if (rc == 0 && cfx_policy_forward(cp, &io, st) != CFX_OK) rc = 1;
        if (rc) {
            fprintf(stderr, "cfx: %s\n", cfx_last_error());
            break;
        }
        refcl_k_compare<<<grid, block, 0, st>>>(logits, b_a, ref_val, d_lav, ref_act, cfx_act, n, d_fmax, d_counts);
        /* the env advances with the actions of the path under test */
        step_mark_kernel<<<grid, block, 0, st>>>(g, cfx_act, rewards, done[t & 1], reset_list, reset_ctrl, n);
        refcl_k_count_done<<<grid, block, 0, st>>>(done[t & 1], n, d_counts);
        int rwgrid = (n + RESET_WARP_BLOCK / 32 - 1) / (RESET_WARP_BLOCK / 32);
        if (rwgrid > 512) rwgrid = 512;
        reset_warp_ctr_kernel<<<rwgrid, RESET_WARP_BLOCK, 0, st>>>(g, reset_list, reset_ctrl, n, seed, step_ctr);
        bump_ctr_kernel<<<1, 1, 0, st>>>(step_ctr);
        RC_CHECK(cudaGetLastError());
        if ((t & 15) == 15) RC_CHECK(cudaStreamSynchronize(st));
    }
    RC_CHECK(cudaStreamSynchronize(st));
    if (rc == 0 && cfx_policy_check(cp, st) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        rc = 1;
    }
    unsigned fm[4];
    unsigned long long cn[4];
    RC_CHECK(cudaMemcpy(fm, d_fmax, sizeof(fm), cudaMemcpyDeviceToHost));
    RC_CHECK(cudaMemcpy(cn, d_counts, sizeof(cn), cudaMemcpyDeviceToHost));
    const double total = (double)n * (double)steps;
    float f0, f1, f2;
    memcpy(&f0, &fm[0], 4); memcpy(&f1, &fm[1], 4); memcpy(&f2, &fm[2], 4);
    out[0] = f0; out[1] = f1; out[2] = (double)cn[0] / total; out[3] = (double)cn[1] / total;
    out[4] = (double)cn[2]; out[5] = f2; out[6] = total;
    if (cp) cfx_policy_destroy(cp);
    cudaFree(arena); cudaFree(d_params); cudaFree(h0); cudaFree(h1); cudaFree(pre); cudaFree(logits);
    cudaFree(ref_state); cudaFree(ref_lp); cudaFree(ref_val); cudaFree(rewards); cudaFree(term); cudaFree(d_lav);
    cudaFree(ref_act); cudaFree(cfx_act); cudaFree(reset_list); cudaFree(reset_ctrl); cudaFree(done[0]);
    cudaFree(done[1]); cudaFree(rec); cudaFree(step_ctr); cudaFree(d_fmax); cudaFree(d_counts);
    cudaStreamDestroy(st);
    cublasDestroy(blas);
    return rc;
}

/* ---- record write: record_obs_kernel (craftax_classic.cu:1884-1890) beside cfx_classic_record_obs ----
 * The view is filled from the reference's EnvSoA (the binding a maintainer would add).  The env
 * plays `steps` steps with uniformly random actions and auto-reset; the records of every step
 * are written with both kernels and compared byte by byte; both kernels are then timed.
 * out[0] differing bytes, out[1] rows compared, out[2] / out[3] ms per call of the reference's /
 * the library's kernel (CUDA events, 20 calls), out[4] rows of the last step with a mob in view,
 * out[5] episode ends. */
static void refcl_fill_view(const EnvSoA& g, cfx_classic_env_view* w) {
    memset(w, 0, sizeof(*w));
    w->num_envs = g.n;
    w->map_packed = g.map_packed; w->map_stride = MAP_PACKED_SIZE;
    w->player_r = g.player_r; w->player_c = g.player_c; w->player_dir = g.player_dir;
    w->health = g.health; w->food = g.food; w->drink = g.drink; w->energy = g.energy;
    w->is_sleeping = g.is_sleeping; w->inv = g.inv;
    w->zombie_r = g.zombie_r; w->zombie_c = g.zombie_c; w->zombie_mask = g.zombie_mask;
    w->cow_r = g.cow_r; w->cow_c = g.cow_c; w->cow_mask = g.cow_mask;
    w->skel_r = g.skel_r; w->skel_c = g.skel_c; w->skel_mask = g.skel_mask;
    w->arrow_r = g.arrow_r; w->arrow_c = g.arrow_c; w->arrow_mask = g.arrow_mask;
    w->light_level = g.light_level;
}
__global__ void refcl_k_random_actions(int32_t* act, int n, uint32_t seed, uint32_t step) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    uint32_t h = seed * 0x9E3779B1u ^ (step + 0x7F4A7C15u) * 0x85EBCA77u ^ ((uint32_t)e + 0x165667B1u) * 0xC2B2AE3Du;
    h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
    act[e] = (int32_t)(h % NUM_ACTIONS);
}
__global__ void refcl_k_count_diff(const uint8_t* a, const uint8_t* b, size_t bytes, unsigned long long* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long d = 0;
    for (; i < bytes; i += (size_t)gridDim.x * blockDim.x) d += a[i] != b[i];
    if (d) atomicAdd(out, d);
}
int refcl_record_parity(int n, int steps, unsigned long long seed, double* out) {
    cudaStream_t st;
    RC_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    uint8_t* arena;
    RC_CHECK(cudaMalloc(&arena, soa_bytes(n)));
    RC_CHECK(cudaMemset(arena, 0, soa_bytes(n)));
    EnvSoA g = carve_soa(arena, n);
    cfx_classic_env_view w;
    refcl_fill_view(g, &w);
    const size_t bytes = (size_t)n * OBS_DIM_COMPACT;
    uint8_t *ra, *rb;
    int8_t* done;
    int32_t *act, *reset_list, *reset_ctrl;
    float* rewards;
    uint64_t* step_ctr;
    unsigned long long* d_cnt;
    RC_CHECK(cudaMalloc(&ra, bytes)); RC_CHECK(cudaMalloc(&rb, bytes));
    RC_CHECK(cudaMalloc(&done, (size_t)n)); RC_CHECK(cudaMalloc(&act, (size_t)n * 4));
    RC_CHECK(cudaMalloc(&reset_list, (size_t)n * 4)); RC_CHECK(cudaMalloc(&reset_ctrl, 8));
    RC_CHECK(cudaMalloc(&rewards, (size_t)n * 4)); RC_CHECK(cudaMalloc(&step_ctr, 8));
    RC_CHECK(cudaMemset(step_ctr, 0, 8));
    RC_CHECK(cudaMalloc(&d_cnt, 4 * sizeof(unsigned long long)));
    RC_CHECK(cudaMemset(d_cnt, 0, 4 * sizeof(unsigned long long)));
    int dev = 0, rc = 0;
    RC_CHECK(cudaGetDevice(&dev));
    const int block = 256, grid = (n + block - 1) / block;
    {
        int wgrid = (int)(((size_t)n * 32 + RESET_WARP_BLOCK - 1) / RESET_WARP_BLOCK);
        reset_all_warp_kernel<<<wgrid, RESET_WARP_BLOCK, 0, st>>>(g, n, seed);
        RC_CHECK(cudaGetLastError());
    }
    for (int t = 0; t < steps && rc == 0; t++) {
        RC_CHECK(cudaMemsetAsync(ra, 0xCD, bytes, st));
        RC_CHECK(cudaMemsetAsync(rb, 0xEF, bytes, st));
        record_obs_kernel<<<grid, block, 0, st>>>(g, ra, n);
        if (cfx_classic_record_obs(dev, &w, rb, n, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); rc = 1; break; }
        refcl_k_count_diff<<<1024, 256, 0, st>>>(ra, rb, bytes, d_cnt);
        RC_CHECK(cudaMemsetAsync(reset_ctrl, 0, 8, st));
        refcl_k_random_actions<<<grid, block, 0, st>>>(act, n, (uint32_t)seed, (uint32_t)t);
        step_mark_kernel<<<grid, block, 0, st>>>(g, act, rewards, done, reset_list, reset_ctrl, n);
        refcl_k_count_done<<<grid, block, 0, st>>>(done, n, d_cnt);   /* counts[2] += episode ends */
        int rwgrid = (n + RESET_WARP_BLOCK / 32 - 1) / (RESET_WARP_BLOCK / 32);
        if (rwgrid > 512) rwgrid = 512;
        reset_warp_ctr_kernel<<<rwgrid, RESET_WARP_BLOCK, 0, st>>>(g, reset_list, reset_ctrl, n, seed, step_ctr);
        bump_ctr_kernel<<<1, 1, 0, st>>>(step_ctr);
        RC_CHECK(cudaGetLastError());
        if ((t & 15) == 15) RC_CHECK(cudaStreamSynchronize(st));
    }
    RC_CHECK(cudaStreamSynchronize(st));
    float ms_ref = 0.f, ms_cfx = 0.f;
    if (rc == 0) {
        cudaEvent_t a, b;
        RC_CHECK(cudaEventCreate(&a)); RC_CHECK(cudaEventCreate(&b));
        for (int k = 0; k < 3; k++) record_obs_kernel<<<grid, block, 0, st>>>(g, ra, n);
        RC_CHECK(cudaEventRecord(a, st));
        for (int k = 0; k < 20; k++) record_obs_kernel<<<grid, block, 0, st>>>(g, ra, n);
        RC_CHECK(cudaEventRecord(b, st));
        RC_CHECK(cudaStreamSynchronize(st));
        RC_CHECK(cudaEventElapsedTime(&ms_ref, a, b));
        for (int k = 0; k < 3; k++) cfx_classic_record_obs(dev, &w, rb, n, st);
        RC_CHECK(cudaEventRecord(a, st));
        for (int k = 0; k < 20; k++) cfx_classic_record_obs(dev, &w, rb, n, st);
        RC_CHECK(cudaEventRecord(b, st));
        RC_CHECK(cudaStreamSynchronize(st));
        RC_CHECK(cudaEventElapsedTime(&ms_cfx, a, b));
        cudaEventDestroy(a); cudaEventDestroy(b);
    }
    unsigned long long cn[4];
    RC_CHECK(cudaMemcpy(cn, d_cnt, sizeof(cn), cudaMemcpyDeviceToHost));
    {
        uint8_t* h = (uint8_t*)malloc(bytes);
        RC_CHECK(cudaMemcpy(h, rb, bytes, cudaMemcpyDeviceToHost));
        double with_mob = 0;
        for (int e = 0; e < n; e++) {
            int any = 0;
            for (int c = 0; c < OBS_MAP_CELLS; c++) any |= h[(size_t)e * OBS_DIM_COMPACT + OBS_MAP_CELLS + c] != 0;
            with_mob += any;
        }
        out[4] = with_mob;
        free(h);
    }
    out[0] = (double)cn[0]; out[1] = (double)n * steps; out[2] = ms_ref / 20.0; out[3] = ms_cfx / 20.0;
    out[5] = (double)cn[2];
    cudaFree(arena); cudaFree(ra); cudaFree(rb); cudaFree(done); cudaFree(act); cudaFree(reset_list);
    cudaFree(reset_ctrl); cudaFree(rewards); cudaFree(step_ctr); cudaFree(d_cnt);
    cudaStreamDestroy(st);
    return rc;
}

/* ---- whole classic rollouts: the step of main_classic.cu's Rollout::step (:439-474) built from the
 * reference's own kernels, and the same step with the policy half (and the record write) taken
 * from the library.  mode 0: reference (encode_env_warp_kernel, record_obs_kernel, cublasSgemm in
 * its TF32 math mode :283 + mingru_epi_fwd_kernel per layer, value_sample_kernel); mode 1:
 * record_obs_kernel + cfx_policy_forward; mode 2: cfx_classic_record_obs + cfx_policy_forward.
 * The env half (step_mark_kernel, reset_warp_ctr_kernel, bump_ctr_kernel) is the reference's in
 * every mode.  Random-init weights of the reference's own layout are passed in; returns
 * env-steps per second over `steps` steps after 3 warm-up steps (CUDA events, eager launches). */
double refcl_rollout_sps(int n, int steps, unsigned long long seed, const float* host_params, int mode,
                         int precision) {
    cublasHandle_t blas;
    RC_BLAS(cublasCreate(&blas));
    RC_BLAS(cublasSetMathMode(blas, CUBLAS_TF32_TENSOR_OP_MATH));
    cudaStream_t st;
    RC_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    RC_BLAS(cublasSetStream(blas, st));
    uint8_t* arena;
    RC_CHECK(cudaMalloc(&arena, soa_bytes(n)));
    RC_CHECK(cudaMemset(arena, 0, soa_bytes(n)));
    EnvSoA g = carve_soa(arena, n);
    float* d_params;
    RC_CHECK(cudaMalloc(&d_params, (size_t)PARAM_COUNT * sizeof(float)));
    RC_CHECK(cudaMemcpy(d_params, host_params, (size_t)PARAM_COUNT * sizeof(float), cudaMemcpyHostToDevice));
    const float* W_enc = d_params + PARAM_W_ENC;
    const float* b_enc = d_params + PARAM_B_ENC;
    const float* W_gru = d_params + PARAM_W_GRU;
    const float* W_a = d_params + PARAM_W_A;
    const float* b_a = d_params + PARAM_B_A;
    const float* W_v = d_params + PARAM_W_V;
    const float* b_v = d_params + PARAM_B_V;
    const size_t hn = (size_t)HIDDEN * n;
    float *h_enc, *hout[2], *h3, *pre, *logits, *h_state, *lp, *val, *rewards, *term;
    int32_t *act, *reset_list, *reset_ctrl;
    int8_t* done[2];
    uint8_t* rec;
    uint64_t* step_ctr;
    RC_CHECK(cudaMalloc(&h_enc, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&hout[0], hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&hout[1], hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&h3, hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&pre, (size_t)GRU_OUT * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&logits, (size_t)NUM_ACTIONS * n * sizeof(float)));
    RC_CHECK(cudaMalloc(&h_state, (size_t)GRU_LAYERS * hn * sizeof(float)));
    RC_CHECK(cudaMemset(h_state, 0, (size_t)GRU_LAYERS * hn * sizeof(float)));
    RC_CHECK(cudaMalloc(&lp, (size_t)n * 4)); RC_CHECK(cudaMalloc(&val, (size_t)n * 4));
    RC_CHECK(cudaMalloc(&rewards, (size_t)n * 4)); RC_CHECK(cudaMalloc(&term, (size_t)n * 4));
    RC_CHECK(cudaMalloc(&act, (size_t)n * 4)); RC_CHECK(cudaMalloc(&reset_list, (size_t)n * 4));
    RC_CHECK(cudaMalloc(&reset_ctrl, 8));
    RC_CHECK(cudaMalloc(&done[0], (size_t)n)); RC_CHECK(cudaMalloc(&done[1], (size_t)n));
    RC_CHECK(cudaMalloc(&rec, (size_t)n * OBS_DIM_COMPACT));
    RC_CHECK(cudaMalloc(&step_ctr, 8));
    RC_CHECK(cudaMemset(step_ctr, 0, 8));
    int dev = 0;
    RC_CHECK(cudaGetDevice(&dev));
    cfx_policy* cp = NULL;
    cfx_classic_env_view w;
    refcl_fill_view(g, &w);
    if (mode != 0 && (cfx_policy_create_classic(&cp, dev, n, HIDDEN, GRU_LAYERS, NUM_ACTIONS, precision) != CFX_OK ||
                      cfx_policy_set_weights(cp, d_params, PARAM_COUNT, 1) != CFX_OK)) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        return -1.0;
    }
    const int block = 256, grid = (n + block - 1) / block;
    const int wgrid = (int)(((size_t)n * 32 + block - 1) / block);
    {
        int rgrid = (int)(((size_t)n * 32 + RESET_WARP_BLOCK - 1) / RESET_WARP_BLOCK);
        reset_all_warp_kernel<<<rgrid, RESET_WARP_BLOCK, 0, st>>>(g, n, seed);
        RC_CHECK(cudaGetLastError());
        RC_CHECK(cudaStreamSynchronize(st));
    }
    const float one = 1.0f, zero = 0.0f;
    const int warm = 3;
    cudaEvent_t ea, eb;
    RC_CHECK(cudaEventCreate(&ea)); RC_CHECK(cudaEventCreate(&eb));
    for (int t = 0; t < warm + steps; t++) {
        if (t == warm) RC_CHECK(cudaEventRecord(ea, st));
        const int8_t* prev = (t == 0) ? NULL : done[(t - 1) & 1];
        RC_CHECK(cudaMemsetAsync(reset_ctrl, 0, 8, st));
        if (mode == 0) {
            encode_env_warp_kernel<<<wgrid, block, 0, st>>>(g, W_enc, b_enc, h_enc, n);
            record_obs_kernel<<<grid, block, 0, st>>>(g, rec, n);
            const float* x = h_enc;
            for (int l = 0; l < GRU_LAYERS; l++) {
                RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, GRU_OUT, n, HIDDEN, &one,
                                    W_gru + (size_t)l * GRU_OUT * HIDDEN, HIDDEN, x, HIDDEN, &zero, pre, GRU_OUT));
                float* xn = (l < GRU_LAYERS - 1) ? hout[l & 1] : h3;
                mingru_epi_fwd_kernel<<<(int)((hn + block - 1) / block), block, 0, st>>>(
                    pre, x, h_state + (size_t)l * hn, xn, NULL, prev, n);
                x = xn;
            }
            RC_BLAS(cublasSgemm(blas, CUBLAS_OP_T, CUBLAS_OP_N, NUM_ACTIONS, n, HIDDEN, &one, W_a, HIDDEN, h3, HIDDEN,
                                &zero, logits, NUM_ACTIONS));
            value_sample_kernel<<<grid, block, 0, st>>>(h3, logits, b_a, W_v, b_v, act, lp, val, n, seed, step_ctr);
        } else {
            if (mode == 2) {
                if (cfx_classic_record_obs(dev, &w, rec, n, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); return -1.0; }
            } else {
                record_obs_kernel<<<grid, block, 0, st>>>(g, rec, n);
            }
            if (prev && cfx_classic_done_to_terminals(dev, prev, term, n, st) != CFX_OK) return -1.0;
            cfx_forward_io io;
            memset(&io, 0, sizeof(io));
            io.records = rec;
            io.prev_terminals = prev ? term : NULL;
            io.actions = act; io.logprobs = lp; io.values = val;
            io.seed = seed;
            if (cfx_policy_forward(cp, &io, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); return -1.0; }
        }
        step_mark_kernel<<<grid, block, 0, st>>>(g, act, rewards, done[t & 1], reset_list, reset_ctrl, n);
        int rwgrid = (n + RESET_WARP_BLOCK / 32 - 1) / (RESET_WARP_BLOCK / 32);
        if (rwgrid > 512) rwgrid = 512;
        reset_warp_ctr_kernel<<<rwgrid, RESET_WARP_BLOCK, 0, st>>>(g, reset_list, reset_ctrl, n, seed, step_ctr);
        bump_ctr_kernel<<<1, 1, 0, st>>>(step_ctr);
        RC_CHECK(cudaGetLastError());
    }
    RC_CHECK(cudaEventRecord(eb, st));
    RC_CHECK(cudaStreamSynchronize(st));
    float ms = 0.f;
    RC_CHECK(cudaEventElapsedTime(&ms, ea, eb));
    if (cp && cfx_policy_check(cp, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); ms = -1.f; }
    if (cp) cfx_policy_destroy(cp);
    cudaEventDestroy(ea); cudaEventDestroy(eb);
    cudaFree(arena); cudaFree(d_params); cudaFree(h_enc); cudaFree(hout[0]); cudaFree(hout[1]); cudaFree(h3);
    cudaFree(pre); cudaFree(logits); cudaFree(h_state); cudaFree(lp); cudaFree(val); cudaFree(rewards); cudaFree(term);
    cudaFree(act); cudaFree(reset_list); cudaFree(reset_ctrl); cudaFree(done[0]); cudaFree(done[1]); cudaFree(rec);
    cudaFree(step_ctr);
    cudaStreamDestroy(st);
    cublasDestroy(blas);
    return ms > 0.f ? (double)n * (double)steps / ((double)ms * 1e-3) : -1.0;
}
#endif

} /* extern "C" */
