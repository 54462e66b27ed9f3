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

} /* extern "C" */
