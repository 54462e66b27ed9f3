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
#include <stddef.h>
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

/* The reference's own checkpoint writer and reader (cu_save_weights / cu_load_weights,
 * :12248-12293) on the fp32-only policy; the loaded arena is mirrored into the bf16 policy. */
void refcu_save_cfw1(void* h, const char* path) {
    refcu* r = (refcu*)h;
    cu_save_weights(&r->pol[1], path);
}

int refcu_load_cfw1(void* h, const char* path) {
    refcu* r = (refcu*)h;
    g_gemm_bf16 = 0;
    if (cu_load_weights(&r->pol[1], path) != 0) return 1;
    g_gemm_bf16 = 1;
    return cu_load_weights(&r->pol[0], path);
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

/* ---- whole rollouts on the GPU (reference env kernels + a policy forward) ----
 * refcu_rollout_sps: the reference's own `run` loop (cu_rollout_step_plain, :12089) with its
 *   default GEMM mode (bf16 at >= 4096 envs on sm_100, :11325), CUDA-graph replay as in
 *   cu_run_rollout_bench (:12127); returns env-steps per second measured with CUDA events.
 * refcu_env_only_sps: env kernels only (what remains of a step when the policy costs nothing).
 * refcu_rollout_swap_sps (built with -DCFX_REF_WITH_CFX): the same loop with the policy half of
 *   cu_rollout_step (:12022-12050: expand, encoder GEMM, bias, GRU chain, head GEMM, sampler)
 *   replaced by one cfx_policy_forward call - the binding a maintainer would add. */
static double refcu_time_steps(CuPolicy* p, int n, int iters, int graph, void (*step)(void*), void* ctx) {
    int warm = iters / 20 > 10 ? 10 : (iters / 20 > 0 ? iters / 20 : 1);
    for (int k = 0; k < warm; k++) step(ctx);
    CU_CHECK(cudaStreamSynchronize(p->stream));
    cudaGraph_t g = NULL;
    cudaGraphExec_t ge = NULL;
    if (graph) {
        CU_CHECK(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeGlobal));
        step(ctx);
        CU_CHECK(cudaStreamEndCapture(p->stream, &g));
        if (cudaGraphInstantiate(&ge, g, NULL, NULL, 0) != cudaSuccess) { cudaGetLastError(); ge = NULL; }
    }
    cudaEvent_t a, b;
    CU_CHECK(cudaEventCreate(&a));
    CU_CHECK(cudaEventCreate(&b));
    CU_CHECK(cudaEventRecord(a, p->stream));
    for (int k = 0; k < iters; k++) {
        if (ge) CU_CHECK(cudaGraphLaunch(ge, p->stream));
        else step(ctx);
    }
    CU_CHECK(cudaEventRecord(b, p->stream));
    CU_CHECK(cudaStreamSynchronize(p->stream));
    float ms = 0.f;
    CU_CHECK(cudaEventElapsedTime(&ms, a, b));
    cudaEventDestroy(a); cudaEventDestroy(b);
    if (ge) cudaGraphExecDestroy(ge);
    if (g) cudaGraphDestroy(g);
    return (double)n * (double)iters / ((double)ms * 1e-3);
}

typedef struct { CuVec* v; CuPolicy* p; uint64_t seed; void* cfx; } refcu_roll;

static void refcu_step_reference(void* c) {
    refcu_roll* r = (refcu_roll*)c;
    cu_rollout_step_plain(r->v, r->p, r->seed);
}

static void refcu_step_env_only(void* c) {
    refcu_roll* r = (refcu_roll*)c;
    CuVec* v = r->v; CuPolicy* p = r->p;
    int n = v->num_envs;
    cudaStream_t st = p->stream;
    CU_CHECK(cudaMemsetAsync(v->d_reset_count, 0, sizeof(int), st));
    CU_CHECK(cudaMemsetAsync(v->d_spawn_count, 0, sizeof(int), st));
    cu_launch_step_run(v->d_envs, n, v->d_resets, NULL, st);
    int tail_blocks = (n * 32 + 255) / 256;
    if (tail_blocks > 512) tail_blocks = 512;
    k_spawn_tail<<<tail_blocks, 256, 0, st>>>();
    if (v->lazy) cu_launch_reset_list_warp(v->d_envs, v->d_resets, n, st);
    else k_reset_list<<<(n + 63) / 64, 64, 0, st>>>(v->d_envs, v->d_resets);
    CU_CHECK(cudaGetLastError());
}

double refcu_rollout_sps(int n, int iters, unsigned long long seed, int graph) {
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    cu_policy_init(&p, n);
    refcu_roll r = {&v, &p, seed, NULL};
    double sps = refcu_time_steps(&p, n, iters, graph, refcu_step_reference, &r);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return sps;
}

double refcu_env_only_sps(int n, int iters, unsigned long long seed, int graph) {
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    cu_policy_init(&p, n);
    CU_CHECK(cudaMemset(v.d_actions, 0, (size_t)n * sizeof(float)));   /* every env plays action 0 */
    refcu_roll r = {&v, &p, seed, NULL};
    double sps = refcu_time_steps(&p, n, iters, graph, refcu_step_env_only, &r);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return sps;
}

#ifdef CFX_REF_WITH_CFX
#include "cfx.h"
static void refcu_fill_view(const CuVec* v, cfx_env_view* w);
/* non-NULL: the record write of the swapped step is cfx_record_obs on this view instead of
 * k_record_obs (set by refcu_rollout_swap_sps for its swap_record mode) */
static const cfx_env_view* g_refcu_record_view = NULL;
static void refcu_step_swapped(void* c) {
    refcu_roll* r = (refcu_roll*)c;
    CuVec* v = r->v; CuPolicy* p = r->p;
    int n = v->num_envs;
    cudaStream_t st = p->stream;
    if (g_refcu_record_view != NULL) {
        int dev = 0;
        CU_CHECK(cudaGetDevice(&dev));
        if (cfx_record_obs(dev, g_refcu_record_view, p->rec, n, NULL, st) != CFX_OK) {
            fprintf(stderr, "cfx: %s\n", cfx_last_error());
            exit(1);
        }
    } else {
        k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(p->rec, n);
    }
    CU_CHECK(cudaMemsetAsync(v->d_reset_count, 0, sizeof(int), st));
    CU_CHECK(cudaMemsetAsync(v->d_spawn_count, 0, sizeof(int), st));
    cfx_forward_io io;
    memset(&io, 0, sizeof(io));
    io.records = p->rec;
    io.prev_terminals = v->d_terminals;
    io.env_actions = v->d_actions;
    io.actions = p->d_act; io.logprobs = p->d_logprob; io.values = p->d_value;
    io.seed = r->seed;
    io.bump_step = 1;
    if (cfx_policy_forward((cfx_policy*)r->cfx, &io, st) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        exit(1);
    }
    cu_launch_step_run(v->d_envs, n, v->d_resets, NULL, st);
    int tail_blocks = (n * 32 + 255) / 256;
    if (tail_blocks > 512) tail_blocks = 512;
    k_spawn_tail<<<tail_blocks, 256, 0, st>>>();
    if (v->lazy) cu_launch_reset_list_warp(v->d_envs, v->d_resets, n, st);
    else k_reset_list<<<(n + 63) / 64, 64, 0, st>>>(v->d_envs, v->d_resets);
    CU_CHECK(cudaGetLastError());
}

/* precision: a CFX_PREC_* code.  The reference policy is created too (its init allocates the
 * record scratch and the sampler outputs the loop writes); its weights are handed over. */
double refcu_rollout_swap2_sps(int n, int iters, unsigned long long seed, int graph, int precision,
                               int swap_record);
double refcu_rollout_swap_sps(int n, int iters, unsigned long long seed, int graph, int precision) {
    return refcu_rollout_swap2_sps(n, iters, seed, graph, precision, 0);
}
/* swap_record != 0: the record write is taken from the library too (cfx_record_obs) */
double refcu_rollout_swap2_sps(int n, int iters, unsigned long long seed, int graph, int precision,
                               int swap_record) {
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    cu_policy_init(&p, n);
    cfx_env_view view;
    refcu_fill_view(&v, &view);
    g_refcu_record_view = swap_record ? &view : NULL;
    int dev = 0;
    CU_CHECK(cudaGetDevice(&dev));
    cfx_policy* cp = NULL;
    if (cfx_policy_create(&cp, dev, n, CF_NN_HIDDEN, CF_NN_LAYERS, CRAFTAX_NUM_ACTIONS, precision) != CFX_OK ||
        cfx_policy_set_weights(cp, p.params, CF_NN_PARAM_COUNT, 1) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        exit(1);
    }
    CU_CHECK(cudaDeviceSynchronize());
    refcu_roll r = {&v, &p, seed, cp};
    double sps = refcu_time_steps(&p, n, iters, graph, refcu_step_swapped, &r);
    g_refcu_record_view = NULL;
    cfx_policy_destroy(cp);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return sps;
}
/* ---- the reference's `play` mode on the new handle ----
 * cu_run_play (:12383-12447) replays a trained policy and writes, per step, one level/done byte
 * per env (k_dump_levels) and the frames of the recorded envs (k_record_frames, CfFrame
 * :12296-12309) for its offline renderer.  refcu_play runs the same loop with the same,
 * unmodified recorders and the same file formats; swapped = 0 calls cu_run_play itself,
 * swapped = 1 takes the step from refcu_step_swapped (policy half = cfx_policy_forward at
 * `precision`) with the weights loaded from the same CFW1 file by cfx_policy_load_cfw1. */
int refcu_frame_bytes(void) { return (int)sizeof(CfFrame); }
int refcu_frame_action_offset(void) { return (int)offsetof(CfFrame, action); }

int refcu_play(int n, int steps, unsigned long long seed, const char* load_path, int swapped, int precision,
               int record_env, int record_n, int record_every, const char* frames_path,
               const char* levels_path) {
    if (!swapped)
        return cu_run_play(n, steps, seed, load_path, record_env, record_n, record_every, frames_path, levels_path);
    if (record_every < 1) record_every = 1;
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    cu_policy_init(&p, n);   /* record row and sampler outputs of the loop */
    int dev = 0;
    CU_CHECK(cudaGetDevice(&dev));
    cfx_policy* cp = NULL;
    if (cfx_policy_create(&cp, dev, n, CF_NN_HIDDEN, CF_NN_LAYERS, CRAFTAX_NUM_ACTIONS, precision) != CFX_OK ||
        cfx_policy_load_cfw1(cp, load_path) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        return 1;
    }
    int rec0 = 0, recn = 0;
    if (record_n > 0) recn = record_n < n ? record_n : n;
    else if (record_env >= 0 && record_env < n) { rec0 = record_env; recn = 1; }
    FILE* ff = (frames_path && recn) ? fopen(frames_path, "wb") : NULL;
    FILE* lf = levels_path ? fopen(levels_path, "wb") : NULL;
    CfFrame* d_frame = NULL;
    CfFrame* h_frame = NULL;
    uint8_t* d_lv = NULL;
    uint8_t* h_lv = (uint8_t*)malloc((size_t)n);
    if (recn) {
        CU_CHECK(cudaMalloc(&d_frame, (size_t)recn * sizeof(CfFrame)));
        h_frame = (CfFrame*)malloc((size_t)recn * sizeof(CfFrame));
    }
    CU_CHECK(cudaMalloc(&d_lv, (size_t)n));
    refcu_roll r = {&v, &p, seed, cp};
    for (int step = 0; step < steps; step++) {
        refcu_step_swapped(&r);
        if (lf) {
            k_dump_levels<<<(n + 255) / 256, 256, 0, p.stream>>>(v.d_envs, v.d_terminals, n, d_lv);
            CU_CHECK(cudaMemcpyAsync(h_lv, d_lv, (size_t)n, cudaMemcpyDeviceToHost, p.stream));
        }
        int rec_now = ff && step % record_every == 0;
        if (rec_now) {
            k_record_frames<<<recn, 256, 0, p.stream>>>(v.d_envs, rec0, p.d_act, v.d_rewards, v.d_terminals,
                                                        d_frame);
            CU_CHECK(cudaMemcpyAsync(h_frame, d_frame, (size_t)recn * sizeof(CfFrame), cudaMemcpyDeviceToHost,
                                     p.stream));
        }
        CU_CHECK(cudaStreamSynchronize(p.stream));
        if (lf) fwrite(h_lv, 1, (size_t)n, lf);
        if (rec_now) fwrite(h_frame, sizeof(CfFrame), (size_t)recn, ff);
    }
    if (ff) fclose(ff);
    if (lf) fclose(lf);
    int rc = cfx_policy_check(cp, p.stream) == CFX_OK ? 0 : 1;
    cudaFree(d_frame); cudaFree(d_lv);
    free(h_frame); free(h_lv);
    cfx_policy_destroy(cp);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return rc;
}

/* ---- lock-step rollout: the reference's CUDA env, driven by this library's forward, with the
 * reference's strict-fp32 cuBLAS pipeline consuming the same records beside it ----
 * Protocol of the reference's runverify (:12501-12507, :12545-12603): the env advances with
 * the actions of the path under test (cfx_policy_forward at `precision`); at every step both
 * forwards read the same record row (written on the device by k_record_obs) and the same
 * prev_terminals.  sync_state = 0: both keep their own recurrent state for the whole rollout
 * (free-running); 1: the reference's state is overwritten with this library's before every
 * step, so the figures measure one forward.  The comparison runs on the device every step.
 * out[0] max |dlogit| (reference logits with their bias added), out[1] max |dvalue|,
 * out[2] fraction of env-steps with the same greedy action, out[3] with the same sampled action
 * (same Philox draw on both sides), out[4] episode ends seen, out[5] max |logit|,
 * out[6] env-steps compared.  Returns 0, or 1 when a cfx call failed (message on stderr). */
__global__ void refcu_k_compare(const float* __restrict__ ref_logits, const float* __restrict__ b_a,
                                const float* __restrict__ b_v, const float* __restrict__ cfx_lav,
                                const int* __restrict__ ref_act, const int* __restrict__ cfx_act,
                                const float* __restrict__ terminals, int n, unsigned* fmax,
                                unsigned long long* counts) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const float* r = ref_logits + (size_t)e * CF_NN_AV;
    const float* c = cfx_lav + (size_t)e * CF_NN_AV;
    float dmax = 0.f, lmax = 0.f, rbest = 0.f, cbest = 0.f;
    int ra = 0, ca = 0;
    for (int a = 0; a < CRAFTAX_NUM_ACTIONS; a++) {
        const float rl = r[a] + b_a[a], cl = c[a];
        dmax = fmaxf(dmax, fabsf(rl - cl));
        lmax = fmaxf(lmax, fabsf(rl));
        if (a == 0 || rl > rbest) { rbest = rl; ra = a; }
        if (a == 0 || cl > cbest) { cbest = cl; ca = a; }
    }
    const float dv = fabsf(r[CRAFTAX_NUM_ACTIONS] + b_v[0] - c[CRAFTAX_NUM_ACTIONS]);
    atomicMax(&fmax[0], __float_as_uint(dmax));   /* non-negative floats order like their bits */
    atomicMax(&fmax[1], __float_as_uint(dv));
    atomicMax(&fmax[2], __float_as_uint(lmax));
    if (ra == ca) atomicAdd(&counts[0], 1ULL);
    if (ref_act[e] == cfx_act[e]) atomicAdd(&counts[1], 1ULL);
    if (terminals[e] != 0.0f) atomicAdd(&counts[2], 1ULL);
}

int refcu_lockstep(int n, int steps, unsigned long long seed, const float* host_arena, int precision,
                   int sync_state, double* out) {
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    /* The first cu_ensure_blas() call reads CF_GEMM_BF16 from the environment (bf16 when it is
     * unset, :11309-11310) and would undo a mode chosen before it: initialise first, then
     * select the fp32 pipeline, and again after cu_policy_init (whose auto-gate may change it). */
    cu_ensure_blas();
    g_gemm_bf16 = 0;
    cu_policy_init(&p, n);   /* record row, sampler outputs; also the reference fp32 pipeline */
    g_gemm_bf16 = 0;
    refcu_h2d(p.params, host_arena, (size_t)CF_NN_PARAM_COUNT * sizeof(float));
    cu_params_refresh_bf16(&p, p.stream);
    cu_pack_wav(&p, p.stream);
    CUBLAS_CHECK(cublasSetMathMode(g_blas, CUBLAS_DEFAULT_MATH));
    int dev = 0;
    CU_CHECK(cudaGetDevice(&dev));
    cfx_policy* cp = NULL;
    float* d_lav = NULL; int* d_cact = NULL; unsigned* d_fmax = NULL; unsigned long long* d_counts = NULL;
    CU_CHECK(cudaMalloc(&d_lav, (size_t)n * CF_NN_AV * sizeof(float)));
    CU_CHECK(cudaMalloc(&d_cact, (size_t)n * sizeof(int)));
    CU_CHECK(cudaMalloc(&d_fmax, 4 * sizeof(unsigned)));
    CU_CHECK(cudaMalloc(&d_counts, 4 * sizeof(unsigned long long)));
    CU_CHECK(cudaMemset(d_fmax, 0, 4 * sizeof(unsigned)));
    CU_CHECK(cudaMemset(d_counts, 0, 4 * sizeof(unsigned long long)));
    int rc = 0;
    if (cfx_policy_create(&cp, dev, n, CF_NN_HIDDEN, CF_NN_LAYERS, CRAFTAX_NUM_ACTIONS, precision) != CFX_OK ||
        cfx_policy_set_weights(cp, p.params, CF_NN_PARAM_COUNT, 1) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        rc = 1;
    }
    CU_CHECK(cudaDeviceSynchronize());
    refcu r;
    memset(&r, 0, sizeof(r));
    r.n = n;
    cudaStream_t st = p.stream;
    const size_t state_bytes = (size_t)CF_NN_LAYERS * CF_NN_HIDDEN * n * sizeof(float);
    for (int t = 0; t < steps && rc == 0; t++) {
        k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(p.rec, n);
        CU_CHECK(cudaMemsetAsync(v.d_reset_count, 0, sizeof(int), st));
        CU_CHECK(cudaMemsetAsync(v.d_spawn_count, 0, sizeof(int), st));
        if (sync_state)
            CU_CHECK(cudaMemcpyAsync(p.h_state, cfx_policy_state(cp), state_bytes, cudaMemcpyDeviceToDevice, st));
        /* reference fp32 pipeline: its sampler output goes to p.d_act, its env-action slot to a sink */
        refcu_enqueue(&r, &p, p.rec, v.d_terminals, seed, p.xobs);
        k_bump_ctr<<<1, 1, 0, st>>>(p.step_ctr);
        /* path under test: fills the env's action slots */
        cfx_forward_io io;
        memset(&io, 0, sizeof(io));
        io.records = p.rec;
        io.prev_terminals = v.d_terminals;
        io.env_actions = v.d_actions;
        io.actions = d_cact;
        io.logits_av = d_lav;
        io.seed = seed;
        io.bump_step = 1;
        if (cfx_policy_forward(cp, &io, st) != CFX_OK) {
            fprintf(stderr, "cfx: %s\n", cfx_last_error());
            rc = 1;
            break;
        }
        refcu_k_compare<<<(n + 255) / 256, 256, 0, st>>>(p.logits, p.w.b_a, p.w.b_v, d_lav, p.d_act, d_cact,
                                                         v.d_terminals, n, d_fmax, d_counts);
        cu_launch_step_run(v.d_envs, n, v.d_resets, NULL, st);
        int tail_blocks = (n * 32 + 255) / 256;
        if (tail_blocks > 512) tail_blocks = 512;
        k_spawn_tail<<<tail_blocks, 256, 0, st>>>();
        if (v.lazy) cu_launch_reset_list_warp(v.d_envs, v.d_resets, n, st);
        else k_reset_list<<<(n + 63) / 64, 64, 0, st>>>(v.d_envs, v.d_resets);
        CU_CHECK(cudaGetLastError());
        if ((t & 15) == 15) CU_CHECK(cudaStreamSynchronize(st));
    }
    CU_CHECK(cudaStreamSynchronize(st));
    if (rc == 0 && cfx_policy_check(cp, st) != CFX_OK) {
        fprintf(stderr, "cfx: %s\n", cfx_last_error());
        rc = 1;
    }
    unsigned fm[4]; unsigned long long cn[4];
    CU_CHECK(cudaMemcpy(fm, d_fmax, sizeof(fm), cudaMemcpyDeviceToHost));
    CU_CHECK(cudaMemcpy(cn, d_counts, sizeof(cn), cudaMemcpyDeviceToHost));
    const double total = (double)n * (double)steps;
    float f0, f1, f2;
    memcpy(&f0, &fm[0], 4); memcpy(&f1, &fm[1], 4); memcpy(&f2, &fm[2], 4);
    out[0] = f0; out[1] = f1; out[2] = (double)cn[0] / total; out[3] = (double)cn[1] / total;
    out[4] = (double)cn[2]; out[5] = f2; out[6] = total;
    CUBLAS_CHECK(cublasSetMathMode(g_blas, CUBLAS_TF32_TENSOR_OP_MATH));
    if (cp) cfx_policy_destroy(cp);
    cudaFree(d_lav); cudaFree(d_cact); cudaFree(d_fmax); cudaFree(d_counts);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return rc;
}

/* ---- record write: k_record_obs (:9284-9297) beside cfx_record_obs ----
 * refcu_fill_view describes the reference's device state to the library without naming its
 * structs (the binding a maintainer would add): the SoA field pointers are read back from the
 * g_cf_* symbols cu_vec_init set (:10762-10775), the byte maps are located with offsetof.
 * refcu_record_parity plays `steps` steps with uniformly random actions, writing the records of
 * every step with both kernels and counting the bytes that differ; it then overwrites the
 * fields the record reads with random values (`fuzz` rounds: positions on and off the map,
 * mob slots of every level, type ids in and out of range, random light and block bytes) and
 * compares again: the writer is a pure function of that memory.  It also times both kernels. */
static void refcu_fill_view(const CuVec* v, cfx_env_view* w) {
    memset(w, 0, sizeof(*w));
    w->num_envs = v->num_envs;
    w->state_base = (const uint8_t*)v->d_states;
    w->state_stride = sizeof(CraftaxState);
    w->map_offset = offsetof(CraftaxWorldState, map);
    w->item_map_offset = offsetof(CraftaxWorldState, item_map);
    w->light_map_offset = offsetof(CraftaxWorldState, light_map);
#define REFCU_VIEW(f, T) { void* q = NULL; CU_CHECK(cudaMemcpyFromSymbol(&q, g_cf_##f, sizeof(q))); w->f = (const T*)q; }
    REFCU_VIEW(player_position, int32_t) REFCU_VIEW(player_level, int32_t) REFCU_VIEW(player_direction, int32_t)
    REFCU_VIEW(player_health, float) REFCU_VIEW(player_food, int32_t) REFCU_VIEW(player_drink, int32_t)
    REFCU_VIEW(player_energy, int32_t) REFCU_VIEW(player_mana, int32_t) REFCU_VIEW(is_sleeping, uint8_t)
    REFCU_VIEW(is_resting, uint8_t) REFCU_VIEW(player_xp, int32_t) REFCU_VIEW(player_dexterity, int32_t)
    REFCU_VIEW(player_strength, int32_t) REFCU_VIEW(player_intelligence, int32_t) REFCU_VIEW(inv_wood, int32_t)
    REFCU_VIEW(inv_stone, int32_t) REFCU_VIEW(inv_coal, int32_t) REFCU_VIEW(inv_iron, int32_t)
    REFCU_VIEW(inv_diamond, int32_t) REFCU_VIEW(inv_sapling, int32_t) REFCU_VIEW(inv_pickaxe, int32_t)
    REFCU_VIEW(inv_sword, int32_t) REFCU_VIEW(inv_bow, int32_t) REFCU_VIEW(inv_arrows, int32_t)
    REFCU_VIEW(inv_torches, int32_t) REFCU_VIEW(inv_ruby, int32_t) REFCU_VIEW(inv_sapphire, int32_t)
    REFCU_VIEW(inv_books, int32_t) REFCU_VIEW(inv_armour, int32_t) REFCU_VIEW(inv_potions, int32_t)
    REFCU_VIEW(learned_spells, uint8_t) REFCU_VIEW(sword_enchantment, int32_t) REFCU_VIEW(bow_enchantment, int32_t)
    REFCU_VIEW(armour_enchantments, int32_t) REFCU_VIEW(boss_timesteps_to_spawn_this_round, int32_t)
    REFCU_VIEW(light_level, float) REFCU_VIEW(monsters_killed, int32_t) REFCU_VIEW(mob_position, int32_t)
    REFCU_VIEW(mob_mask, uint8_t) REFCU_VIEW(mob_type_id, int32_t)
#undef REFCU_VIEW
}

static __device__ __forceinline__ uint32_t refcu_hash(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t h = a * 0x9E3779B1u ^ (b + 0x7F4A7C15u) * 0x85EBCA77u ^ (c + 0x165667B1u) * 0xC2B2AE3Du;
    h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
    return h;
}
__global__ void refcu_k_random_actions(float* actions, int n, uint32_t seed, uint32_t step) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) actions[e] = (float)(refcu_hash(seed, step, (uint32_t)e) % CRAFTAX_NUM_ACTIONS);
}
__global__ void refcu_k_skip_flags(uint8_t* flags, int n, uint32_t seed) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) flags[e] = (uint8_t)(refcu_hash(seed, 77u, (uint32_t)e) % 3u == 0u);
}
__global__ void refcu_k_count_diff(const uint8_t* a, const uint8_t* b, size_t bytes, unsigned long long* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long d = 0;
    for (; i < bytes; i += (size_t)gridDim.x * blockDim.x) d += a[i] != b[i];
    if (d) atomicAdd(out, d);
}
/* overwrites what the record reads: one thread per env (round r of the fuzz) */
__global__ void refcu_k_fuzz_state(cfx_env_view w, uint32_t seed, uint32_t r) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = w.num_envs;
    if (e >= n) return;
    uint32_t k = 0;
    auto rnd = [&](uint32_t mod) { return refcu_hash(seed + r * 977u, k++, (uint32_t)e) % mod; };
    auto I = [&](const int32_t* f, int i) -> int32_t& { return const_cast<int32_t*>(f)[(size_t)i * n + e]; };
    auto B = [&](const uint8_t* f, int i) -> uint8_t& { return const_cast<uint8_t*>(f)[(size_t)i * n + e]; };
    auto F = [&](const float* f, int i) -> float& { return const_cast<float*>(f)[(size_t)i * n + e]; };
    const int level = (int)rnd(CRAFTAX_WG_NUM_LEVELS);
    I(w.player_level, 0) = level;
    I(w.player_position, 0) = (int)rnd(CRAFTAX_WG_MAP_SIZE);
    I(w.player_position, 1) = (int)rnd(CRAFTAX_WG_MAP_SIZE);
    I(w.player_direction, 0) = (int)rnd(6);
    F(w.player_health, 0) = (float)rnd(100) * 0.125f;
    const int32_t* small[] = {w.player_food, w.player_drink, w.player_energy, w.player_mana, w.player_xp,
                              w.player_dexterity, w.player_strength, w.player_intelligence, w.inv_pickaxe,
                              w.inv_sword, w.inv_bow, w.inv_books, w.sword_enchantment, w.bow_enchantment};
    for (int i = 0; i < 14; i++) I(small[i], 0) = (int)rnd(10);
    const int32_t* counts[] = {w.inv_wood, w.inv_stone, w.inv_coal, w.inv_iron, w.inv_diamond, w.inv_sapling,
                               w.inv_arrows, w.inv_torches, w.inv_ruby, w.inv_sapphire};
    for (int i = 0; i < 10; i++) I(counts[i], 0) = (int)rnd(100);
    for (int i = 0; i < 4; i++) { I(w.inv_armour, i) = (int)rnd(3); I(w.armour_enchantments, i) = (int)rnd(3); }
    for (int i = 0; i < 6; i++) I(w.inv_potions, i) = (int)rnd(30);
    B(w.is_sleeping, 0) = (uint8_t)rnd(2); B(w.is_resting, 0) = (uint8_t)rnd(2);
    B(w.learned_spells, 0) = (uint8_t)rnd(2); B(w.learned_spells, 1) = (uint8_t)rnd(2);
    I(w.boss_timesteps_to_spawn_this_round, 0) = (int)rnd(5) - 2;
    F(w.light_level, 0) = (float)rnd(1000) * 0.001f;
    for (int l = 0; l < CRAFTAX_WG_NUM_LEVELS; l++) I(w.monsters_killed, l) = (int)rnd(16);
    /* mobs of every class, level and slot: near the player, sometimes off the view or off the map */
    const int pr = I(w.player_position, 0), pc = I(w.player_position, 1);
    for (int m = 0; m < 5 * CRAFTAX_WG_NUM_LEVELS * 3; m++) {
        I(w.mob_type_id, m) = (int)rnd(CRAFTAX_WG_NUM_MOB_TYPES + 2) - 1;
        B(w.mob_mask, m) = (uint8_t)(rnd(4) != 0);
        I(w.mob_position, 2 * m) = pr + (int)rnd(13) - 6;
        I(w.mob_position, 2 * m + 1) = pc + (int)rnd(15) - 7;
    }
    /* the three byte maps of the player's level around the player */
    uint8_t* blk = const_cast<uint8_t*>(w.state_base) + (size_t)e * w.state_stride;
    for (int dr = -6; dr <= 6; dr++)
        for (int dc = -7; dc <= 7; dc++) {
            const int rr = pr + dr, cc = pc + dc;
            if (rr < 0 || rr >= CRAFTAX_WG_MAP_SIZE || cc < 0 || cc >= CRAFTAX_WG_MAP_SIZE) continue;
            const size_t o = ((size_t)level * CRAFTAX_WG_MAP_SIZE + rr) * CRAFTAX_WG_MAP_SIZE + cc;
            blk[w.map_offset + o] = (uint8_t)rnd(40);
            blk[w.item_map_offset + o] = (uint8_t)rnd(6);
            blk[w.light_map_offset + o] = (uint8_t)rnd(26);
        }
}

/* out[0] differing bytes over all compared rows, out[1] rows compared, out[2] / out[3] ms per call
 * of k_record_obs / cfx_record_obs at n envs (CUDA events, 20 calls each), out[4] rows with a
 * visible mob among the compared ones (coverage), out[5] differing bytes of the list variant,
 * out[6] differing bytes with skip flags on every third env (skipped rows keep their bytes). */
int refcu_record_parity(int n, int steps, int fuzz, unsigned long long seed, double* out) {
    CuVec v; CuPolicy p;
    cu_vec_init(&v, n, seed);
    cu_policy_init(&p, n);
    cudaStream_t st = p.stream;
    int dev = 0;
    CU_CHECK(cudaGetDevice(&dev));
    cfx_env_view w;
    refcu_fill_view(&v, &w);
    uint8_t *ra = NULL, *rb = NULL;
    unsigned long long* d_cnt = NULL;
    const size_t bytes = (size_t)n * CF_TRAIN_OBS;
    CU_CHECK(cudaMalloc(&ra, bytes)); CU_CHECK(cudaMalloc(&rb, bytes));
    CU_CHECK(cudaMalloc(&d_cnt, 4 * sizeof(unsigned long long)));
    CU_CHECK(cudaMemset(d_cnt, 0, 4 * sizeof(unsigned long long)));
    int rc = 0;
    double rows = 0;
    auto compare = [&]() {
        CU_CHECK(cudaMemsetAsync(ra, 0xCD, bytes, st));
        CU_CHECK(cudaMemsetAsync(rb, 0xEF, bytes, st));
        k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(ra, n);
        if (cfx_record_obs(dev, &w, rb, n, NULL, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); rc = 1; }
        refcu_k_count_diff<<<1024, 256, 0, st>>>(ra, rb, bytes, d_cnt);
        rows += n;
    };
    for (int t = 0; t < steps && rc == 0; t++) {
        compare();
        refcu_k_random_actions<<<(n + 255) / 256, 256, 0, st>>>(v.d_actions, n, (uint32_t)seed, (uint32_t)t);
        refcu_roll r = {&v, &p, seed, NULL};
        refcu_step_env_only(&r);
        if ((t & 15) == 15) CU_CHECK(cudaStreamSynchronize(st));
    }
    /* the list variant on the last step's reset list (the envs that were just reset) */
    if (rc == 0) {
        CU_CHECK(cudaMemsetAsync(ra, 0xCD, bytes, st));
        CU_CHECK(cudaMemsetAsync(rb, 0xCD, bytes, st));
        k_record_obs_list<<<128, 256, 0, st>>>(ra, v.d_resets);
        if (cfx_record_obs_list(dev, &w, rb, v.d_resets, (int)sizeof(CraftaxResetRec), v.d_reset_count, st) != CFX_OK) {
            fprintf(stderr, "cfx: %s\n", cfx_last_error()); rc = 1;
        }
        refcu_k_count_diff<<<1024, 256, 0, st>>>(ra, rb, bytes, d_cnt + 1);
    }
    for (int r = 0; r < fuzz && rc == 0; r++) {
        refcu_k_fuzz_state<<<(n + 127) / 128, 128, 0, st>>>(w, (uint32_t)seed, (uint32_t)r);
        compare();
    }
    /* the skip flags: rows whose flag is set keep their bytes in both */
    if (rc == 0) {
        uint8_t* flags = NULL;
        CU_CHECK(cudaMalloc(&flags, (size_t)n));
        refcu_k_skip_flags<<<(n + 255) / 256, 256, 0, st>>>(flags, n, (uint32_t)seed);
        CU_CHECK(cudaMemsetAsync(ra, 0xCD, bytes, st));
        CU_CHECK(cudaMemsetAsync(rb, 0xCD, bytes, st));
        k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(ra, n, flags);
        if (cfx_record_obs(dev, &w, rb, n, flags, st) != CFX_OK) { fprintf(stderr, "cfx: %s\n", cfx_last_error()); rc = 1; }
        refcu_k_count_diff<<<1024, 256, 0, st>>>(ra, rb, bytes, d_cnt + 2);
        CU_CHECK(cudaStreamSynchronize(st));
        cudaFree(flags);
    }
    CU_CHECK(cudaStreamSynchronize(st));
    /* timing, on the last state */
    float ms_ref = 0.f, ms_cfx = 0.f;
    {
        cudaEvent_t a, b;
        CU_CHECK(cudaEventCreate(&a)); CU_CHECK(cudaEventCreate(&b));
        for (int k = 0; k < 3; k++) k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(ra, n);
        CU_CHECK(cudaEventRecord(a, st));
        for (int k = 0; k < 20; k++) k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(ra, n);
        CU_CHECK(cudaEventRecord(b, st));
        CU_CHECK(cudaStreamSynchronize(st));
        CU_CHECK(cudaEventElapsedTime(&ms_ref, a, b));
        for (int k = 0; k < 3; k++) cfx_record_obs(dev, &w, rb, n, NULL, st);
        CU_CHECK(cudaEventRecord(a, st));
        for (int k = 0; k < 20; k++) cfx_record_obs(dev, &w, rb, n, NULL, st);
        CU_CHECK(cudaEventRecord(b, st));
        CU_CHECK(cudaStreamSynchronize(st));
        CU_CHECK(cudaEventElapsedTime(&ms_cfx, a, b));
        cudaEventDestroy(a); cudaEventDestroy(b);
    }
    /* coverage: rows of the last comparison with a mob byte set */
    unsigned long long cn[4];
    CU_CHECK(cudaMemcpy(cn, d_cnt, sizeof(cn), cudaMemcpyDeviceToHost));
    {
        uint8_t* h = (uint8_t*)malloc(bytes);
        CU_CHECK(cudaMemcpy(h, rb, bytes, cudaMemcpyDeviceToHost));
        double with_mob = 0;
        for (int e = 0; e < n; e++) {
            int any = 0;
            for (int c = 0; c < 99 && !any; c++)
                for (int ch = 3; ch < 8; ch++) any |= h[(size_t)e * CF_TRAIN_OBS + c * 8 + ch] != 0;
            with_mob += any;
        }
        out[4] = with_mob;
        free(h);
    }
    out[0] = (double)cn[0]; out[1] = rows; out[2] = ms_ref / 20.0; out[3] = ms_cfx / 20.0; out[5] = (double)cn[1]; out[6] = (double)cn[2];
    cudaFree(ra); cudaFree(rb); cudaFree(d_cnt);
    cu_policy_free(&p);
    cu_vec_free(&v);
    return rc;
}

/* ---- a state of the reference's CUDA env, its records, and the view on it, handed to the caller ----
 * refcu_record_session_open plays `steps` steps with random actions, optionally randomises the
 * state `fuzz` times (refcu_k_fuzz_state), writes the records with k_record_obs into
 * records_host [n][996] and copies the filled cfx_env_view into view_out; the env stays alive
 * until refcu_record_session_close, so that the caller can read the state through the view's
 * device pointers (to run a CPU restatement of the record write on the very same state). */
static CuVec g_sess_v;
static CuPolicy g_sess_p;
static int g_sess_open = 0;
int refcu_record_session_open(int n, int steps, int fuzz, unsigned long long seed, void* view_out,
                              size_t view_bytes, uint8_t* records_host) {
    if (g_sess_open || view_bytes != sizeof(cfx_env_view)) return 1;
    cu_vec_init(&g_sess_v, n, seed);
    cu_policy_init(&g_sess_p, n);
    g_sess_open = 1;
    cudaStream_t st = g_sess_p.stream;
    cfx_env_view w;
    refcu_fill_view(&g_sess_v, &w);
    for (int t = 0; t < steps; t++) {
        refcu_k_random_actions<<<(n + 255) / 256, 256, 0, st>>>(g_sess_v.d_actions, n, (uint32_t)seed, (uint32_t)t);
        refcu_roll r = {&g_sess_v, &g_sess_p, seed, NULL};
        refcu_step_env_only(&r);
        if ((t & 15) == 15) CU_CHECK(cudaStreamSynchronize(st));
    }
    for (int r = 0; r < fuzz; r++)
        refcu_k_fuzz_state<<<(n + 127) / 128, 128, 0, st>>>(w, (uint32_t)seed, (uint32_t)r);
    uint8_t* d_rec = NULL;
    const size_t bytes = (size_t)n * CF_TRAIN_OBS;
    CU_CHECK(cudaMalloc(&d_rec, bytes));
    k_record_obs<<<(int)(((size_t)n * 32 + 255) / 256), 256, 0, st>>>(d_rec, n);
    CU_CHECK(cudaGetLastError());
    CU_CHECK(cudaStreamSynchronize(st));
    CU_CHECK(cudaMemcpy(records_host, d_rec, bytes, cudaMemcpyDeviceToHost));
    cudaFree(d_rec);
    memcpy(view_out, &w, sizeof(w));
    return 0;
}
void refcu_record_session_close(void) {
    if (!g_sess_open) return;
    cu_policy_free(&g_sess_p);
    cu_vec_free(&g_sess_v);
    g_sess_open = 0;
}
#endif


} /* extern "C" */
