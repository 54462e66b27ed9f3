/*
 * The reference's own CUDA policy forward behind a C ABI (TEST AND BASELINE
 * INFRASTRUCTURE; compiled only where the reference sources are present, into
 * oracle/_ref/, never committed).
 *
 * The reference keeps everything `static` in craftax_full.cu and offers
 * -DCRAFTAX_CU_LIB to drop main() so that another translation unit can
 * #include it (craftax_full.cu:13937-13941).  This file does exactly that
 * (path given with -DCFX_REF_CU=\"...\") and exports wrappers that run the
 * reference's UNMODIFIED kernels and cuBLAS wrappers on caller-provided
 * records, weights and state:
 *   batched path  k_expand_obs -> encoder GEMM -> k_add_bias (the body of
 *                 cu_encode_step after the record write, :11954-11962) ->
 *                 cu_gru_chain (:11978) -> head GEMM (:12040-12045) ->
 *                 k_value_sample (:9714), in its bf16 / TF32 / strict-fp32 modes;
 *   scalar path   k_policy_ref_l3 (:9778), the reference's own fp32 yardstick.
 * Uses: pinning the CPU oracle and the fused kernel against reference outputs
 * on the same GPU, and timing the reference's cuBLAS pipeline beside ours.
 */
#define CRAFTAX_CU_LIB 1
#include CFX_REF_CU

enum { REFCU_BF16 = 0, REFCU_TF32 = 1, REFCU_FP32 = 2 };

typedef struct {
    int n;
    CuPolicy pol[2];  /* [0] allocated with bf16 mirrors, [1] fp32-only */
    float* ref_state; /* scalar kernel's private [L][H][n] state */
    float* ref_h3;    /* [n][H] */
    float* zeros;     /* [n] zero terminals, used when the caller passes none: the reference
                         kernels read prev_terminals unconditionally */
} refcu;

/* Host-to-device copy that has LANDED when it returns.  A pageable cudaMemcpy returns once
 * the data is staged; the reference's policy streams are non-blocking, so work enqueued on
 * them next would not wait for the DMA (it would repack or read stale weights). */
static void refcu_h2d(void* dst, const void* src, size_t bytes) {
    CU_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    CU_CHECK(cudaDeviceSynchronize());
}

static CuPolicy* refcu_pick(refcu* r, int mode) {
    g_gemm_bf16 = (mode == REFCU_BF16) ? 1 : 0;
    CUBLAS_CHECK(cublasSetMathMode(
        g_blas, mode == REFCU_FP32 ? CUBLAS_DEFAULT_MATH : CUBLAS_TF32_TENSOR_OP_MATH));
    return &r->pol[mode == REFCU_BF16 ? 0 : 1];
}

extern "C" {

int refcu_layers(void) { return CF_NN_LAYERS; }
int refcu_hidden(void) { return CF_NN_HIDDEN; }
int refcu_param_count(void) { return CF_NN_PARAM_COUNT; }

void* refcu_create(int n) {
    refcu* r = (refcu*)calloc(1, sizeof(refcu));
    r->n = n;
    setenv("CF_GEMM_BF16", "1", 1); /* explicit setting: disables the small-n auto-gate */
    cu_ensure_blas();
    g_gemm_bf16 = 1;
    cu_policy_init(&r->pol[0], n);
    g_gemm_bf16 = 0;
    cu_policy_init(&r->pol[1], n);
    size_t hn = (size_t)CF_NN_HIDDEN * n;
    CU_CHECK(cudaMalloc(&r->ref_state, (size_t)CF_NN_LAYERS * hn * sizeof(float)));
    CU_CHECK(cudaMemset(r->ref_state, 0, (size_t)CF_NN_LAYERS * hn * sizeof(float)));
    CU_CHECK(cudaMalloc(&r->ref_h3, hn * sizeof(float)));
    CU_CHECK(cudaMalloc(&r->zeros, (size_t)n * sizeof(float)));
    CU_CHECK(cudaMemset(r->zeros, 0, (size_t)n * sizeof(float)));
    CU_CHECK(cudaDeviceSynchronize());
    return r;
}

void refcu_destroy(void* h) {
    refcu* r = (refcu*)h;
    cu_policy_free(&r->pol[0]);
    cu_policy_free(&r->pol[1]);
    cudaFree(r->ref_state);
    cudaFree(r->ref_h3);
    cudaFree(r->zeros);
    free(r);
}

/* Same arena into both policies, then the reference's own mirror refresh
 * (cu_params_refresh_bf16 + cu_pack_wav, :11805-11817). */
void refcu_set_weights(void* h, const float* host_arena) {
    refcu* r = (refcu*)h;
    for (int i = 0; i < 2; i++) {
        CuPolicy* p = &r->pol[i];
        refcu_h2d(p->params, host_arena, (size_t)CF_NN_PARAM_COUNT * sizeof(float));
        g_gemm_bf16 = (i == 0);
        cu_params_refresh_bf16(p, p->stream);
        cu_pack_wav(p, p->stream);
        CU_CHECK(cudaStreamSynchronize(p->stream));
    }
}

void refcu_get_weights(void* h, float* host_arena) {
    refcu* r = (refcu*)h;
    CU_CHECK(cudaMemcpy(host_arena, r->pol[1].params, (size_t)CF_NN_PARAM_COUNT * sizeof(float),
                        cudaMemcpyDeviceToHost));
}

/* Live state of the batched path, [L][n][H] (same layout as ours). */
void refcu_set_state(void* h, int mode, const float* host_state) {
    refcu* r = (refcu*)h;
    CuPolicy* p = &r->pol[mode == REFCU_BF16 ? 0 : 1];
    refcu_h2d(p->h_state, host_state, (size_t)CF_NN_LAYERS * CF_NN_HIDDEN * r->n * sizeof(float));
}

void refcu_get_state(void* h, int mode, float* host_state) {
    refcu* r = (refcu*)h;
    CuPolicy* p = &r->pol[mode == REFCU_BF16 ? 0 : 1];
    CU_CHECK(cudaMemcpy(host_state, p->h_state,
                        (size_t)CF_NN_LAYERS * CF_NN_HIDDEN * r->n * sizeof(float),
                        cudaMemcpyDeviceToHost));
}

void refcu_set_step(void* h, unsigned long long step) {
    refcu* r = (refcu*)h;
    for (int i = 0; i < 2; i++)
        refcu_h2d(r->pol[i].step_ctr, &step, sizeof(step));
}

/* Enqueues the batched forward on the policy's stream (no sync). */
static void refcu_enqueue(refcu* r, CuPolicy* p, const uint8_t* d_rec, const float* d_prev_terminals,
                          uint64_t seed, float* d_env_actions) {
    const int n = r->n;
    cudaStream_t st = p->stream;
    k_expand_obs<<<(int)(((size_t)CF_NN_OBS * n + 255) / 256), 256, 0, st>>>(
        d_rec, p->xobs, 0, n, n, n, 0, g_gemm_bf16 ? p->xobs_bf : NULL);
    if (g_gemm_bf16)
        cu_gemm_nn_bf(CF_NN_OBS, n, p->params_bf + CF_NN_W_ENC, p->xobs_bf, CF_NN_OBS_PAD,
                      p->h_enc, st);
    else
        cu_gemm_enc_fwd(n, p->w.W_enc, p->xobs, p->h_enc, st);
    k_add_bias<<<(int)(((size_t)CF_NN_HIDDEN * n + 255) / 256), 256, 0, st>>>(
        p->h_enc, p->w.b_enc, n, g_gemm_bf16 ? p->henc_bf : NULL);
    cu_gru_chain(p, p->h_enc, p->h_state, d_prev_terminals, NULL, p->h3, n, st);
    if (g_gemm_bf16)
        cu_gemm_fwd_bf(CF_NN_AV, n, CF_NN_HIDDEN, p->W_av_bf, p->h3_bf, p->logits, st);
    else
        cu_gemm_fwd(CF_NN_AV, n, CF_NN_HIDDEN, p->W_av, p->h3, p->logits, st);
    k_value_sample<<<(n + 255) / 256, 256, 0, st>>>(p->logits, p->w.b_a, p->w.b_v, d_env_actions,
                                                    p->d_act, p->d_logprob, p->d_value, n, seed,
                                                    p->step_ctr);
}

/* One batched forward.  Host outputs (any may be NULL): logits [n][44] BEFORE the
 * bias add as the reference stores them, h3 [n][H], actions, logprobs, values. */
void refcu_forward(void* h, int mode, const uint8_t* d_rec, const float* d_prev_terminals,
                   unsigned long long seed, float* d_env_actions, float* logits, float* h3,
                   int* actions, float* logprobs, float* values) {
    refcu* r = (refcu*)h;
    CuPolicy* p = refcu_pick(r, mode);
    const size_t n = r->n;
    if (!d_prev_terminals) d_prev_terminals = r->zeros;
    refcu_enqueue(r, p, d_rec, d_prev_terminals, seed, d_env_actions ? d_env_actions : p->xobs);
    CU_CHECK(cudaGetLastError());
    CU_CHECK(cudaStreamSynchronize(p->stream));
    if (logits) CU_CHECK(cudaMemcpy(logits, p->logits, n * CF_NN_AV * sizeof(float), cudaMemcpyDeviceToHost));
    if (h3) CU_CHECK(cudaMemcpy(h3, p->h3, n * CF_NN_HIDDEN * sizeof(float), cudaMemcpyDeviceToHost));
    if (actions) CU_CHECK(cudaMemcpy(actions, p->d_act, n * sizeof(int), cudaMemcpyDeviceToHost));
    if (logprobs) CU_CHECK(cudaMemcpy(logprobs, p->d_logprob, n * sizeof(float), cudaMemcpyDeviceToHost));
    if (values) CU_CHECK(cudaMemcpy(values, p->d_value, n * sizeof(float), cudaMemcpyDeviceToHost));
}

/* Times `iters` forwards (after `warm` untimed ones) with CUDA events; graph != 0
 * captures one forward and replays it, as the reference's run mode does (:12142-12160).
 * Returns milliseconds per forward. */
float refcu_time_forward(void* h, int mode, const uint8_t* d_rec, const float* d_prev_terminals,
                         int warm, int iters, int graph) {
    refcu* r = (refcu*)h;
    CuPolicy* p = refcu_pick(r, mode);
    float* sink = p->xobs; /* env action slot stand-in */
    if (!d_prev_terminals) d_prev_terminals = r->zeros;
    for (int i = 0; i < warm; i++) {
        refcu_enqueue(r, p, d_rec, d_prev_terminals, 1, sink);
        k_bump_ctr<<<1, 1, 0, p->stream>>>(p->step_ctr);
    }
    CU_CHECK(cudaStreamSynchronize(p->stream));
    cudaGraph_t g = NULL;
    cudaGraphExec_t ge = NULL;
    if (graph) {
        CU_CHECK(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeGlobal));
        refcu_enqueue(r, p, d_rec, d_prev_terminals, 1, sink);
        k_bump_ctr<<<1, 1, 0, p->stream>>>(p->step_ctr);
        CU_CHECK(cudaStreamEndCapture(p->stream, &g));
        if (cudaGraphInstantiate(&ge, g, NULL, NULL, 0) != cudaSuccess) {
            cudaGetLastError();
            ge = NULL;
        }
    }
    cudaEvent_t a, b;
    CU_CHECK(cudaEventCreate(&a));
    CU_CHECK(cudaEventCreate(&b));
    CU_CHECK(cudaEventRecord(a, p->stream));
    for (int i = 0; i < iters; i++) {
        if (ge) {
            CU_CHECK(cudaGraphLaunch(ge, p->stream));
        } else {
            refcu_enqueue(r, p, d_rec, d_prev_terminals, 1, sink);
            k_bump_ctr<<<1, 1, 0, p->stream>>>(p->step_ctr);
        }
    }
    CU_CHECK(cudaEventRecord(b, p->stream));
    CU_CHECK(cudaEventSynchronize(b));
    float ms = 0.0f;
    CU_CHECK(cudaEventElapsedTime(&ms, a, b));
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (ge) cudaGraphExecDestroy(ge);
    if (g) cudaGraphDestroy(g);
    return ms / (float)iters;
}

/* The reference's scalar fp32 policy on records (compact-obs build: its observation
 * pointer is the record array).  State is its private [L][H][n] buffer; set/get below
 * convert from/to the [L][n][H] layout used everywhere else. */
void refcu_scalar_set_state(void* h, const float* host_state_lnh) {
    refcu* r = (refcu*)h;
    const int n = r->n, H = CF_NN_HIDDEN, L = CF_NN_LAYERS;
    float* t = (float*)malloc((size_t)L * H * n * sizeof(float));
    for (int l = 0; l < L; l++)
        for (int e = 0; e < n; e++)
            for (int k = 0; k < H; k++)
                t[((size_t)l * H + k) * n + e] = host_state_lnh[((size_t)l * n + e) * H + k];
    refcu_h2d(r->ref_state, t, (size_t)L * H * n * sizeof(float));
    free(t);
}

void refcu_scalar_get_state(void* h, float* host_state_lnh) {
    refcu* r = (refcu*)h;
    const int n = r->n, H = CF_NN_HIDDEN, L = CF_NN_LAYERS;
    float* t = (float*)malloc((size_t)L * H * n * sizeof(float));
    CU_CHECK(cudaMemcpy(t, r->ref_state, (size_t)L * H * n * sizeof(float), cudaMemcpyDeviceToHost));
    for (int l = 0; l < L; l++)
        for (int e = 0; e < n; e++)
            for (int k = 0; k < H; k++)
                host_state_lnh[((size_t)l * n + e) * H + k] = t[((size_t)l * H + k) * n + e];
    free(t);
}

void refcu_scalar_forward(void* h, const uint8_t* d_rec, const float* d_prev_terminals,
                          unsigned long long seed, float* h3, int* actions, float* logprobs,
                          float* values) {
    refcu* r = (refcu*)h;
    CuPolicy* p = &r->pol[1];
    const size_t n = r->n;
    if (!d_prev_terminals) d_prev_terminals = r->zeros;
    k_policy_ref_l3<<<(r->n + 63) / 64, 64, 0, p->stream>>>(
        p->w, r->ref_state, d_prev_terminals, (const CraftaxObs*)d_rec, p->d_act, p->d_logprob,
        p->d_value, r->ref_h3, r->n, seed, p->step_ctr);
    CU_CHECK(cudaGetLastError());
    CU_CHECK(cudaStreamSynchronize(p->stream));
    if (h3) CU_CHECK(cudaMemcpy(h3, r->ref_h3, n * CF_NN_HIDDEN * sizeof(float), cudaMemcpyDeviceToHost));
    if (actions) CU_CHECK(cudaMemcpy(actions, p->d_act, n * sizeof(int), cudaMemcpyDeviceToHost));
    if (logprobs) CU_CHECK(cudaMemcpy(logprobs, p->d_logprob, n * sizeof(float), cudaMemcpyDeviceToHost));
    if (values) CU_CHECK(cudaMemcpy(values, p->d_value, n * sizeof(float), cudaMemcpyDeviceToHost));
}

} /* extern "C" */
