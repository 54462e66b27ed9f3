// Strict-fp32 forward on CUDA cores (precision CFX_PREC_FP32) plus the
// stand-alone expand / sampler / uniform stages.
//
// Every dot product is accumulated with fmaf in ascending input order, which
// is the order of the reference's scalar policy kernel (k_policy_ref_l3,
// craftax_full.cu:9778-9854); this file is compiled with -fmad=false like the
// reference's full-game build (Makefile:27), so the cell arithmetic rounds at
// the same places.  It is the high-accuracy mode of the library and the
// on-device yardstick for the tensor-core kernel at sizes a CPU cannot check.
#include <cuda_bf16.h>

#include <atomic>

#include "cfx_common.cuh"
#include "cfx_sampler.cuh"
#include "cfx_strict.h"

namespace cfx {

// ---------------------------------------------------------------- expand
// features[e][f] = (float)rec[e][f] for f < 792, raw fp32 bits for the tail
// (k_expand_obs, craftax_full.cu:10028-10053).  One thread per output element;
// consecutive threads write consecutive floats.
__global__ void k_expand(const uint8_t* __restrict__ rec, float* __restrict__ out, int n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * kObs) return;
    int f = (int)(idx % kObs);
    size_t e = idx / kObs;
    const uint8_t* r = rec + e * kRec;
    float x;
    if (f < kMap) {
        x = (float)r[f];
    } else {
        // records are 4-byte aligned (996 = 4 * 249, 792 = 4 * 198)
        x = *reinterpret_cast<const float*>(r + kMap + 4 * (f - kMap));
    }
    out[idx] = x;
}

// ---------------------------------------------------------------- encoder
// h_enc[e][k] = b_enc[k] + sum_f x[e][f] * W_enc[f][k], ascending f.
// Block = H threads (one per unit) x ENC_ENVS envs; the records of the tile are
// expanded chunk-wise into shared memory as fp32, transposed to [f][e] so the
// inner loop reads x by broadcast and W_enc rows coalesced.
constexpr int ENC_ENVS = 32;
constexpr int ENC_FCHUNK = 64;

__global__ void k_encoder_fp32(const uint8_t* __restrict__ rec, const float* __restrict__ W_enc,
                               const float* __restrict__ b_enc, float* __restrict__ h_out,
                               int n, int H) {
    __shared__ float xs[ENC_FCHUNK][ENC_ENVS + 1];
    const int e0 = blockIdx.x * ENC_ENVS;
    const int k = threadIdx.x;  // unit
    float acc[ENC_ENVS];
    const float b = b_enc[k];
#pragma unroll
    for (int e = 0; e < ENC_ENVS; e++) acc[e] = b;
    for (int f0 = 0; f0 < kObs; f0 += ENC_FCHUNK) {
        const int fc = min(ENC_FCHUNK, kObs - f0);
        __syncthreads();
        for (int i = threadIdx.x; i < ENC_ENVS * ENC_FCHUNK; i += blockDim.x) {
            int e = i / ENC_FCHUNK, f = i % ENC_FCHUNK;
            float x = 0.0f;
            if (f < fc && e0 + e < n) {
                const uint8_t* r = rec + (size_t)(e0 + e) * kRec;
                int ff = f0 + f;
                x = ff < kMap ? (float)r[ff]
                              : *reinterpret_cast<const float*>(r + kMap + 4 * (ff - kMap));
            }
            xs[f][e] = x;
        }
        __syncthreads();
        for (int f = 0; f < fc; f++) {
            const float w = W_enc[(size_t)(f0 + f) * H + k];
#pragma unroll
            for (int e = 0; e < ENC_ENVS; e++) acc[e] = fmaf(xs[f][e], w, acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < ENC_ENVS; e++)
        if (e0 + e < n) h_out[(size_t)(e0 + e) * H + k] = acc[e];
}

// ---------------------------------------------------------------- classic game
// Record -> 1345 features, reference expand_obs_kernel (craftax_classic.cu:1265-1301).
__global__ void k_classic_expand(const uint8_t* __restrict__ rec, float* __restrict__ out, int n) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const uint8_t* c = rec + (size_t)e * kClassicRec;
    float* o = out + (size_t)e * kClassicObs;
    int k = 0;
    for (int cell = 0; cell < kClassicCells; cell++) {
        const int8_t blk = (int8_t)c[cell];
        for (int b = 0; b < kClassicBlocks; b++) o[k++] = (blk == b) ? 1.0f : 0.0f;
        const uint8_t m = c[kClassicCells + cell];
        for (int j = 0; j < 4; j++) o[k++] = (m & (1 << j)) ? 1.0f : 0.0f;
    }
    int i2 = 2 * kClassicCells;
    for (int j = 0; j < kClassicInv + 4; j++) o[k++] = (float)(int8_t)c[i2++] / 10.0f;
    const int8_t dir = (int8_t)c[i2++];
    for (int d = 1; d <= 4; d++) o[k++] = (dir == d) ? 1.0f : 0.0f;
    const uint8_t sleeping = c[i2++];
    float light;
    memcpy(&light, c + i2, 4);
    o[k++] = light;
    o[k++] = sleeping ? 1.0f : 0.0f;
}

// Gather encoder in the order of the reference's encode_obs_kernel (craftax_classic.cu:1714-1751):
// bias, then per cell the block column and the set mob bits, then the 22 scalar features, every
// term as fmaf(x, W, acc).  One thread per (env, unit); the block's threads read a W_enc row
// coalesced.  Block ids outside [0,16] (never written by the game) are skipped.
__global__ void k_classic_encoder_fp32(const uint8_t* __restrict__ rec, const float* __restrict__ W_enc,
                                       const float* __restrict__ b_enc, float* __restrict__ h_out,
                                       int n, int H) {
    __shared__ uint8_t rs[kClassicRec];
    const int e = blockIdx.x;
    const int k = threadIdx.x;
    for (int i = threadIdx.x; i < kClassicRec; i += blockDim.x) rs[i] = rec[(size_t)e * kClassicRec + i];
    __syncthreads();
    const float* Wk = W_enc + k;
    float hv = b_enc[k];
    for (int cell = 0; cell < kClassicCells; cell++) {
        const int blk = (int8_t)rs[cell];
        if (blk >= 0 && blk < kClassicBlocks)
            hv = fmaf(1.0f, Wk[(size_t)(cell * (kClassicBlocks + 4) + blk) * H], hv);
        const uint8_t m = rs[kClassicCells + cell];
        const int fm = cell * (kClassicBlocks + 4) + kClassicBlocks;
        for (int j = 0; j < 4; j++)
            if (m & (1 << j)) hv = fmaf(1.0f, Wk[(size_t)(fm + j) * H], hv);
    }
    int oi = 2 * kClassicCells;
    int f = kClassicCells * (kClassicBlocks + 4);
    for (int j = 0; j < kClassicInv + 4; j++, f++)
        hv = fmaf((float)(int8_t)rs[oi++] / 10.0f, Wk[(size_t)f * H], hv);
    const int8_t dir = (int8_t)rs[oi++];
    for (int d = 1; d <= 4; d++, f++) hv = fmaf((dir == d) ? 1.0f : 0.0f, Wk[(size_t)f * H], hv);
    const uint8_t sleeping = rs[oi++];
    float light;
    memcpy(&light, rs + oi, 4);
    hv = fmaf(light, Wk[(size_t)f * H], hv);
    f++;
    hv = fmaf(sleeping ? 1.0f : 0.0f, Wk[(size_t)f * H], hv);
    h_out[(size_t)e * H + k] = hv;
}

// r_done int8 flags of the classic rollout (main_classic.cu:436-443) -> the float flags the
// MinGRU kernel takes
__global__ void k_done_to_terminals(const int8_t* __restrict__ done, float* __restrict__ out, int n) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) out[e] = done[e] != 0 ? 1.0f : 0.0f;
}

// ---------------------------------------------------------------- MinGRU layer
// One layer: gate dots (ascending j, fmaf) + cell (k_mingru_epi_fwd,
// craftax_full.cu:9350-9395).  Wt is the layer's gate matrix transposed to
// [H][3H] so that unit-indexed threads read it coalesced.
constexpr int GRU_ENVS = 16;

__device__ __forceinline__ float sigmoid_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float mingru_g_ref(float x) { return x >= 0.0f ? x + 0.5f : sigmoid_ref(x); }

__global__ void k_mingru_fp32(const float* __restrict__ x_in, const float* __restrict__ Wt,
                              float* __restrict__ state, const float* __restrict__ prev_terminals,
                              float* __restrict__ h_out, float* __restrict__ r_state, int r_bf16,
                              int n, int H) {
    extern __shared__ float xs[];  // [GRU_ENVS][H]
    const int e0 = blockIdx.x * GRU_ENVS;
    const int k = threadIdx.x;
    for (int i = threadIdx.x; i < GRU_ENVS * H; i += blockDim.x) {
        int e = i / H;
        xs[i] = (e0 + e < n) ? x_in[(size_t)e0 * H + i] : 0.0f;
    }
    __syncthreads();
    float zh[GRU_ENVS], zg[GRU_ENVS], zp[GRU_ENVS];
#pragma unroll
    for (int e = 0; e < GRU_ENVS; e++) zh[e] = zg[e] = zp[e] = 0.0f;
    for (int j = 0; j < H; j++) {
        const float* wr = Wt + (size_t)j * 3 * H;
        const float wh = wr[k], wg = wr[H + k], wp = wr[2 * H + k];
#pragma unroll
        for (int e = 0; e < GRU_ENVS; e++) {
            const float xv = xs[e * H + j];
            zh[e] = fmaf(wh, xv, zh[e]);
            zg[e] = fmaf(wg, xv, zg[e]);
            zp[e] = fmaf(wp, xv, zp[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < GRU_ENVS; e++) {
        if (e0 + e >= n) break;
        const size_t o = (size_t)(e0 + e) * H + k;
        float st = state[o];
        if (prev_terminals != nullptr && prev_terminals[e0 + e] != 0.0f) st = 0.0f;
        if (r_state != nullptr) {
            if (r_bf16) reinterpret_cast<__nv_bfloat16*>(r_state)[o] = __float2bfloat16(st);
            else r_state[o] = st;
        }
        const float out = st + sigmoid_ref(zg[e]) * (mingru_g_ref(zh[e]) - st);
        const float p = sigmoid_ref(zp[e]);
        h_out[o] = p * out + (1.0f - p) * xs[e * H + k];
        state[o] = out;
    }
}

// ---------------------------------------------------------------- heads
// logits_av[e][a] = bias[a] + sum_j W_av[a][j] * h[e][j] (ascending j); row A
// is the value head.  Accumulator starts at the bias as in the scalar
// reference (craftax_full.cu:9838-9845).
constexpr int HEAD_ENVS = 8;

__global__ void k_heads_fp32(const float* __restrict__ h, const float* __restrict__ W_a,
                             const float* __restrict__ b_a, const float* __restrict__ W_v,
                             const float* __restrict__ b_v, float* __restrict__ logits_av,
                             int n, int H, int A) {
    extern __shared__ float hs[];  // [HEAD_ENVS][H]
    const int e0 = blockIdx.x * HEAD_ENVS;
    for (int i = threadIdx.x; i < HEAD_ENVS * H; i += blockDim.x) {
        int e = i / H;
        hs[i] = (e0 + e < n) ? h[(size_t)e0 * H + i] : 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < HEAD_ENVS * (A + 1); i += blockDim.x) {
        const int e = i / (A + 1), a = i % (A + 1);
        if (e0 + e >= n) continue;
        const float* w = a < A ? W_a + (size_t)a * H : W_v;
        float z = a < A ? b_a[a] : b_v[0];
        const float* hv = hs + e * H;
        for (int j = 0; j < H; j++) z = fmaf(w[j], hv[j], z);
        logits_av[(size_t)(e0 + e) * (A + 1) + a] = z;
    }
}

// ---------------------------------------------------------------- sampler
// One thread per env (k_value_sample, craftax_full.cu:9714-9741); logits
// already carry their biases.
__global__ void k_sample(const float* __restrict__ logits, int ld, int A,
                         const float* __restrict__ uniforms, uint64_t seed, uint64_t env_offset,
                         const unsigned long long* __restrict__ step_ctr, int n,
                         float* __restrict__ env_actions, int32_t* __restrict__ actions,
                         float* __restrict__ logprobs, float* __restrict__ values) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const float* l = logits + (size_t)e * ld;
    float u;
    if (uniforms != nullptr) u = uniforms[e];
    else u = philox_uniform(seed, env_offset + (uint64_t)e, step_ctr ? *step_ctr : 0ULL);
    float lp;
    const int a = sample_action_dyn(l, A, u, &lp);
    if (env_actions) env_actions[e] = (float)a;
    if (actions) actions[e] = a;
    if (logprobs) logprobs[e] = lp;
    if (values) values[e] = l[A];
}

__global__ void k_uniforms(uint64_t seed, uint64_t env_offset, uint64_t step, int n, float* u) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) u[e] = philox_uniform(seed, env_offset + (uint64_t)e, step);
}

__global__ void k_bump(unsigned long long* ctr) { *ctr += 1ULL; }

// Gate matrices transposed for the strict layer kernel: Wt[l][j][r] = W[l][r][j].
__global__ void k_transpose_gates(const float* __restrict__ W, float* __restrict__ Wt, int H, int L) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t per = (size_t)3 * H * H;
    if (idx >= per * L) return;
    size_t l = idx / per, r = (idx % per) / H, j = idx % H;
    Wt[l * per + j * 3 * H + r] = W[idx];
}

// Reference initialiser: U(+-bound) from Philox(seed, subsequence, index)
// (k_nn_init_weights, craftax_full.cu:9123-9131).
__global__ void k_init_uniform(float* w, int count, float bound, uint64_t seed, int subseq) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    curandStatePhilox4_32_10_t st;
    curand_init(seed, (uint64_t)subseq, (uint64_t)i, &st);
    w[i] = (2.0f * curand_uniform(&st) - 1.0f) * bound;
}

// ---------------------------------------------------------------- launchers
int launch_expand(const uint8_t* rec, float* out, int n, cudaStream_t st) {
    size_t total = (size_t)n * kObs;
    k_expand<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(rec, out, n);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_classic_expand(const uint8_t* rec, float* out, int n, cudaStream_t st) {
    k_classic_expand<<<(n + 127) / 128, 128, 0, st>>>(rec, out, n);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_done_to_terminals(const int8_t* done, float* out, int n, cudaStream_t st) {
    k_done_to_terminals<<<(n + 255) / 256, 256, 0, st>>>(done, out, n);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_sample(const float* logits, int ld, int A, const float* u, uint64_t seed,
                  uint64_t env_offset, const unsigned long long* step_ctr, int n,
                  float* env_actions, int32_t* actions, float* logprobs, float* values,
                  cudaStream_t st) {
    k_sample<<<(n + 127) / 128, 128, 0, st>>>(logits, ld, A, u, seed, env_offset, step_ctr, n,
                                              env_actions, actions, logprobs, values);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_uniforms(uint64_t seed, uint64_t env_offset, uint64_t step, int n, float* u, cudaStream_t st) {
    k_uniforms<<<(n + 255) / 256, 256, 0, st>>>(seed, env_offset, step, n, u);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_bump(unsigned long long* ctr, cudaStream_t st) {
    k_bump<<<1, 1, 0, st>>>(ctr);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_transpose_gates(const float* W, float* Wt, int H, int L, cudaStream_t st) {
    size_t total = (size_t)L * 3 * H * H;
    k_transpose_gates<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(W, Wt, H, L);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int launch_init_uniform(float* w, int count, float bound, uint64_t seed, int subseq, cudaStream_t st) {
    k_init_uniform<<<(count + 255) / 256, 256, 0, st>>>(w, count, bound, seed, subseq);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

// Full strict forward.  scratch_h: two [n][H] fp32 buffers; logits_av [n][A+1].
int strict_forward(const StrictArgs& a, cudaStream_t st, int* launches) {
    const int H = a.H, L = a.L, A = a.A, n = a.n;
    const ArenaLayout o = ArenaLayout::make(H, L, A, a.game == CFX_GAME_CLASSIC ? kClassicObs : kObs);
    int cnt = 0;
    if (a.game == CFX_GAME_CLASSIC)
        k_classic_encoder_fp32<<<n, H, 0, st>>>(a.records, a.params + o.w_enc, a.params + o.b_enc,
                                                a.scratch_h[0], n, H);
    else
        k_encoder_fp32<<<(n + ENC_ENVS - 1) / ENC_ENVS, H, 0, st>>>(
            a.records, a.params + o.w_enc, a.params + o.b_enc, a.scratch_h[0], n, H);
    cnt++;
    const float* x = a.scratch_h[0];
    for (int l = 0; l < L; l++) {
        float* out = a.scratch_h[(l + 1) & 1];
        k_mingru_fp32<<<(n + GRU_ENVS - 1) / GRU_ENVS, H, GRU_ENVS * H * sizeof(float), st>>>(
            x, a.gates_t + (size_t)l * 3 * H * H, a.state + (size_t)l * n * H, a.prev_terminals,
            out,
            a.r_state ? reinterpret_cast<float*>(reinterpret_cast<char*>(a.r_state) +
                                                 (size_t)l * n * H * (a.r_state_bf16 ? 2 : 4))
                      : nullptr,
            a.r_state_bf16, n, H);
        cnt++;
        x = out;
    }
    k_heads_fp32<<<(n + HEAD_ENVS - 1) / HEAD_ENVS, 128, HEAD_ENVS * H * sizeof(float), st>>>(
        x, a.params + o.w_a, a.params + o.b_a, a.params + o.w_v, a.params + o.b_v,
        a.logits_av, n, H, A);
    cnt++;
    k_sample<<<(n + 127) / 128, 128, 0, st>>>(a.logits_av, A + 1, A, a.uniforms, a.seed,
                                              a.env_offset, a.step_ctr, n, a.env_actions,
                                              a.actions, a.logprobs, a.values);
    cnt++;
    CFX_CUDA(cudaGetLastError());
    if (launches) *launches = cnt;
    return CFX_OK;
}

}  // namespace cfx

// ---------------------------------------------------------------- allocation-free variant
// Strict fp32 forward whose scratch lives in a fixed device array instead of buffers from
// cudaMalloc.  Meant for hosts that must not allocate once they are running: a rollout
// worker embedded in another runtime that owns the whole device heap and hands out no
// memory, or a latency-bound loop where cudaMalloc's device-wide synchronisation (and its
// chance of failing on a fragmented heap hours into a run) is not acceptable.  Such a caller
// brings its own parameter arena, state, inputs and outputs; everything else is here.
//
// Limits: hidden = 256, layers <= 4, actions <= 63, num_envs <= 1024 (multiple of 32).
// The array (5.5 MB) is resident on every GPU that loads this library until the process
// exits.  All calls share it: two calls that overlap on the GPU (different streams, or
// different host threads) race on it; serialise them.  Nothing in it has to start at zero:
// the transposed gate matrices, both layer buffers and the logits are fully rewritten by
// each call before they are read, so stale contents of an earlier call are harmless.
namespace cfx {
constexpr int kStaticMaxEnvs = 1024, kStaticHidden = 256, kStaticMaxLayers = 4;
constexpr size_t kStaticGates = (size_t)kStaticMaxLayers * 3 * kStaticHidden * kStaticHidden;
constexpr size_t kStaticLayerBuf = (size_t)kStaticMaxEnvs * kStaticHidden;
constexpr size_t kStaticLogits = (size_t)kStaticMaxEnvs * (kMaxActions + 1);
constexpr size_t kStaticFloats = kStaticGates + 2 * kStaticLayerBuf + kStaticLogits;

static __device__ __align__(256) float g_static_scratch[kStaticFloats];

// Device address of the array per device ordinal; in host code the symbol's name is only a
// handle for cudaGetSymbolAddress, never a pointer a kernel could use.  The cache is filled
// once per device (atomic: two host threads may make their first calls together and resolve
// the same address).  It is not invalidated: after cudaDeviceReset the library must be
// reloaded before this entry point is used again.
constexpr int kStaticMaxDevices = 64;
static std::atomic<float*> g_static_scratch_addr[kStaticMaxDevices];
}  // namespace cfx

extern "C" int cfx_strict_forward_static(int device, const float* params, int hidden, int layers,
                                         int num_actions, int num_envs, float* state,
                                         const cfx_forward_io* io, const uint64_t* step_ctr,
                                         void* stream) {
    using namespace cfx;
    CFX_REQUIRE(params && state && io, "cfx_strict_forward_static: NULL argument");
    CFX_REQUIRE(io->records && io->actions, "cfx_strict_forward_static: records/actions is NULL");
    // same rule as cfx_policy_forward; the encoder reads the tail floats of a record as words
    CFX_REQUIRE(((uintptr_t)io->records & 15) == 0,
                "cfx_strict_forward_static: records not 16-byte aligned");
    int ndev = 0;
    CFX_CUDA(cudaGetDeviceCount(&ndev));
    CFX_REQUIRE(device >= 0 && device < ndev && device < kStaticMaxDevices,
                "cfx_strict_forward_static: device %d of %d", device, ndev);
    CFX_REQUIRE(hidden == kStaticHidden,
                "cfx_strict_forward_static: hidden=%d, the fixed scratch is sized for %d", hidden,
                kStaticHidden);
    CFX_REQUIRE(layers >= 1 && layers <= kStaticMaxLayers,
                "cfx_strict_forward_static: layers=%d exceeds the fixed scratch (max %d)", layers,
                kStaticMaxLayers);
    CFX_REQUIRE(num_actions >= 2 && num_actions <= kMaxActions,
                "cfx_strict_forward_static: num_actions=%d out of [2,%d]", num_actions, kMaxActions);
    CFX_REQUIRE(num_envs > 0 && num_envs % 32 == 0 && num_envs <= kStaticMaxEnvs,
                "cfx_strict_forward_static: num_envs=%d must be a multiple of 32 and at most %d "
                "(size of the fixed scratch)", num_envs, kStaticMaxEnvs);
    CFX_GUARD(device);
    cudaStream_t st = (cudaStream_t)stream;
    if (g_static_scratch_addr[device].load(std::memory_order_acquire) == nullptr) {
        // one-time set-up for this device, with it current: resolve the array's device address.
        // It must not happen while the stream is being captured.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) cudaGetLastError();
        CFX_REQUIRE(cap == cudaStreamCaptureStatusNone,
                    "cfx_strict_forward_static: the first call on a device does its set-up and "
                    "must come before any stream capture");
        float* addr = nullptr;
        CFX_CUDA(cudaGetSymbolAddress((void**)&addr, g_static_scratch));
        CFX_REQUIRE(addr != nullptr, "cfx_strict_forward_static: no device address for the scratch");
        g_static_scratch_addr[device].store(addr, std::memory_order_release);
    }
    float* base = g_static_scratch_addr[device].load(std::memory_order_acquire);
    const ArenaLayout o = ArenaLayout::make(hidden, layers, num_actions);
    int rc = launch_transpose_gates(params + o.w_gru, base, hidden, layers, st);
    if (rc) return rc;
    StrictArgs a;
    a.n = num_envs; a.H = hidden; a.L = layers; a.A = num_actions;
    a.params = params;
    a.gates_t = base;
    a.records = io->records;
    a.prev_terminals = io->prev_terminals;
    a.uniforms = io->uniforms;
    a.state = state;
    a.scratch_h[0] = base + kStaticGates;
    a.scratch_h[1] = base + kStaticGates + kStaticLayerBuf;
    a.logits_av = io->logits_av ? io->logits_av : base + kStaticGates + 2 * kStaticLayerBuf;
    a.r_state = io->r_state;
    a.r_state_bf16 = io->r_state_bf16 ? 1 : 0;
    a.env_actions = io->env_actions;
    a.actions = io->actions;
    a.logprobs = io->logprobs;
    a.values = io->values;
    a.seed = io->seed;
    a.env_offset = io->env_offset;
    a.step_ctr = reinterpret_cast<const unsigned long long*>(step_ctr);
    return strict_forward(a, st, nullptr);
}
