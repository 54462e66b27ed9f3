// Fused policy forward for sm_100a: one persistent kernel runs, per 128-env tile,
//   compact records (TMA boxes) -> fp16/bf16 operand rows written straight into tensor
//   memory -> encoder MMA -> MinGRU layers (gate MMA + cell epilogue, activations kept in
//   tensor memory as the next layer's A operand) -> actor/value MMA -> categorical sample.
// HBM traffic is the record, the fp32 recurrent state (read + written through TMA) and the
// outputs; weights stream from L2 through a shared-memory ring as pre-swizzled images.
//
// Replaces, inside cu_rollout_step (craftax_full.cu:12022-12087): k_expand_obs (:10028),
// the encoder GEMM + k_add_bias (:11954-11962), cu_gru_chain (:11978-12014: gate GEMM +
// k_mingru_epi_fwd :9350), the head GEMM (:12040-12045) and k_value_sample (:9714).
//
// Tile-level dataflow (M = 128 envs = the 128 TMEM lanes; thread r of a quarter-warp set
// owns env row r):
//   TMEM columns   gate phase: A0 [0,128) A1 [128,256) (layer inputs, 16-bit packed, ping-pong)
//                              G0 [256,352) G1 [352,448) (gate accumulators of one 32-unit
//                              slice: zh|zg|zp, double buffered)  HEAD [448,496)
//                  encoder phase: operand-chunk ring [0,256) (8 x 32 columns), accumulator
//                              [256,512)
//   shared memory  weight ring 7 x 16 KB | state ring 4 x 16 KB | record ring 4 x 10 KB
//   warps          0 weight loads, 1 MMA issue + TMEM alloc, 2 record loads, 3 state loads,
//                  4 state stores, 5..12 workers (expand, epilogues, sampler)
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "cfx_common.cuh"
#include "cfx_fused.h"
#include "cfx_sampler.cuh"
#include "cfx_tmap.h"
#include "cfx_umma.cuh"

namespace cfx {
using namespace umma;

namespace fused {

constexpr int kH = 256;          // hidden units
constexpr int kA = 43;           // actions
constexpr int kTile = 128;       // envs per tile
constexpr int kMaxLayers = 4;
constexpr int kSliceUnits = 32;  // hidden units per gate slice
constexpr int kSlices = kH / kSliceUnits;  // 8
constexpr int kKBlocks = kH / 64;          // 4 K blocks of 64 per 256-wide operand
constexpr int kEncChunks = 14;   // 12 full map chunks, 1 partial (24 bytes), 1 tail (51 floats)
constexpr int kRecSubs = 16;     // record ring fills per tile: 13 map + 3 tail boxes-sets
constexpr int kHeadN = 48;       // 43 logits + value, padded to a multiple of 16

constexpr int kBSlot = 16384, kNB = 7;
constexpr int kSSlot = 16384, kNS = 4;
constexpr int kRBoxBytes = 32 * 80, kRSlot = 4 * kRBoxBytes, kNR = 4;
constexpr int kAexpSlots = 8;

constexpr int kEncStageBytes = 128 * 128;            // [128 units][64 K] 16-bit
constexpr int kGateStageBytes = 3 * kSliceUnits * 128;  // [96 rows][64 K]
constexpr int kHeadStageBytes = kHeadN * 128;        // [48 rows][64 K]
constexpr int kEncStages = kEncChunks * 2;

__host__ __device__ constexpr size_t image_bytes(int L) {
    return (size_t)kEncStages * kEncStageBytes + (size_t)L * kSlices * kKBlocks * kGateStageBytes +
           (size_t)kKBlocks * kHeadStageBytes;
}

// TMEM columns
constexpr uint32_t kColA0 = 0, kColA1 = 128, kColG0 = 256, kColG1 = 352, kColHead = 448;
constexpr uint32_t kColAexp = 0, kColAcc = 256;

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int kOffB = 0;
constexpr int kOffS = kOffB + kNB * kBSlot;
constexpr int kOffR = kOffS + kNS * kSSlot;
constexpr int kOffBias = kOffR + kNR * kRSlot;     // b_enc[256] fp32, b_av[48] fp32
constexpr int kOffBars = kOffBias + (kH + kHeadN) * 4;
enum Bar {
    B_FULL = 0, B_EMPTY = B_FULL + kNB, S_FULL = B_EMPTY + kNB, S_EMPTY = S_FULL + kNS,
    ST_READY = S_EMPTY + kNS, R_FULL = ST_READY + kNS, R_EMPTY = R_FULL + kNR,
    AEXP_FULL = R_EMPTY + kNR, AEXP_EMPTY = AEXP_FULL + kAexpSlots,
    ACC_FULL = AEXP_EMPTY + kAexpSlots, A_KB = ACC_FULL + 1, G_FULL = A_KB + kKBlocks,
    G_EMPTY = G_FULL + 2, H_FULL = G_EMPTY + 2, NUM_BARS = H_FULL + 1
};
constexpr int kOffMisc = kOffBars + NUM_BARS * 8;  // tmem base, abort flag
constexpr int kSmemBytes = kOffMisc + 16 + 1024;   // + alignment slack

constexpr int kWorkerWarp0 = 5, kNumWarps = 13, kThreads = kNumWarps * 32;

// wait-site codes recorded in the status word when a bounded wait gives up
enum WaitCode : uint32_t {
    W_B_EMPTY = 1, W_B_FULL, W_R_EMPTY, W_R_FULL, W_S_EMPTY, W_S_FULL, W_ST_READY, W_AEXP_EMPTY,
    W_AEXP_FULL, W_ACC_FULL, W_A_KB, W_G_FULL, W_G_EMPTY, W_H_FULL
};

struct Params {
    CUtensorMap rec_map;                 // uint8 [n/4][3984], box 32 x 80
    CUtensorMap state_map[kMaxLayers];   // fp32 [n][256] per layer, box 128 x 32, SWIZZLE_128B
    const uint8_t* image;                // pre-swizzled 16-bit weight stages in consumption order
    const float* params;                 // fp32 arena (biases are read from it)
    const float* prev_terminals;
    const float* uniforms;
    float* env_actions;
    int32_t* actions;
    float* logprobs;
    float* values;
    float* logits_av;
    const unsigned long long* step_ctr;
    uint32_t* status;
    uint64_t seed, env_offset;
    int n, L, num_tiles;
    size_t off_b_enc, off_b_a, off_b_v;
};

// ------------------------------------------------------------------ weight image
// Byte offset of (row, 16-bit K column c in [0,64)) inside a 128-byte-swizzled stage.
__host__ __device__ inline uint32_t sw128_off(uint32_t row, uint32_t byte_col) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((byte_col >> 4) ^ (row & 7)) & 7) << 4) +
           (byte_col & 15);
}

// Encoder K order: K' in [0,800) = the 792 map bytes then 8 zero columns; K' in [800,864) =
// the 51 tail floats then 13 zero columns.  Returns the feature index or -1 for padding.
__host__ __device__ inline int enc_feature(int chunk, int c) {
    if (chunk < 12) return chunk * 64 + c;
    if (chunk == 12) return c < 24 ? 768 + c : -1;
    return c < kTail ? kMap + c : -1;
}

template <typename T16>
__device__ inline T16 to16(float v);
template <>
__device__ inline __half to16<__half>(float v) {
    return __float2half_rn(fminf(fmaxf(v, -65504.0f), 65504.0f));
}
template <>
__device__ inline __nv_bfloat16 to16<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// One thread per 16-bit element of the image.  Stage order = consumption order of the
// kernel: encoder (chunk-major, unit halves), gate layers (layer, slice, K block), head.
template <typename T16>
__global__ void k_pack_image(const float* __restrict__ params, uint8_t* __restrict__ image, int L,
                             size_t off_w_gru, size_t off_w_a, size_t off_w_v) {
    const size_t total = image_bytes(L) / 2;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t byte = idx * 2;
    const size_t enc_bytes = (size_t)kEncStages * kEncStageBytes;
    const size_t gate_bytes = (size_t)L * kSlices * kKBlocks * kGateStageBytes;
    float v = 0.0f;
    uint32_t row, c;
    uint8_t* stage;
    if (byte < enc_bytes) {
        const int s = (int)(byte / kEncStageBytes), e = (int)((byte % kEncStageBytes) / 2);
        row = e / 64; c = e % 64;
        stage = image + (size_t)s * kEncStageBytes;
        const int chunk = s / 2, half = s % 2;
        const int f = enc_feature(chunk, c);
        if (f >= 0) v = params[(size_t)f * kH + half * 128 + row];
    } else if (byte < enc_bytes + gate_bytes) {
        const size_t b = byte - enc_bytes;
        const int s = (int)(b / kGateStageBytes), e = (int)((b % kGateStageBytes) / 2);
        row = e / 64; c = e % 64;
        stage = image + enc_bytes + (size_t)s * kGateStageBytes;
        const int kb = s % kKBlocks, j = (s / kKBlocks) % kSlices, l = s / (kKBlocks * kSlices);
        const int gate = row / kSliceUnits, unit = j * kSliceUnits + row % kSliceUnits;
        v = params[off_w_gru + ((size_t)l * 3 * kH + gate * kH + unit) * kH + kb * 64 + c];
    } else {
        const size_t b = byte - enc_bytes - gate_bytes;
        const int kb = (int)(b / kHeadStageBytes), e = (int)((b % kHeadStageBytes) / 2);
        row = e / 64; c = e % 64;
        stage = image + enc_bytes + gate_bytes + (size_t)kb * kHeadStageBytes;
        if (row < kA) v = params[off_w_a + (size_t)row * kH + kb * 64 + c];
        else if (row == kA) v = params[off_w_v + kb * 64 + c];
    }
    *reinterpret_cast<T16*>(stage + sw128_off(row, c * 2)) = to16<T16>(v);
}

// ------------------------------------------------------------------ small device helpers
template <typename T16>
struct Op16;
template <>
struct Op16<__half> {
    static constexpr uint32_t kFmt = kFmtF16;
    // two floats -> packed pair, `lo` in the low half (even K index)
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    static __device__ __forceinline__ float2 unpack(uint32_t v) {
        __half2 h = *reinterpret_cast<__half2*>(&v);
        return __half22float2(h);
    }
    // four record bytes (integers 0..255, exact in fp16) -> two packed pairs:
    // 0x6400 | b is the fp16 number 1024 + b; subtracting 1024 leaves b exactly.
    static __device__ __forceinline__ void bytes4(uint32_t w, uint32_t& p01, uint32_t& p23) {
        uint32_t a = __byte_perm(w, 0x64646464u, 0x5140);
        uint32_t b = __byte_perm(w, 0x64646464u, 0x7362);
        const uint32_t k = 0x64006400u;
        asm("sub.f16x2 %0, %1, %2;" : "=r"(p01) : "r"(a), "r"(k));
        asm("sub.f16x2 %0, %1, %2;" : "=r"(p23) : "r"(b), "r"(k));
    }
};
template <>
struct Op16<__nv_bfloat16> {
    static constexpr uint32_t kFmt = kFmtBF16;
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    static __device__ __forceinline__ float2 unpack(uint32_t v) {
        return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
    }
    // 0x4B000000 | b is the fp32 number 2^23 + b; integers 0..255 are exact in bf16.
    static __device__ __forceinline__ void bytes4(uint32_t w, uint32_t& p01, uint32_t& p23) {
        const float m = 8388608.0f;
        float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440)) - m;
        float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7441)) - m;
        float f2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7442)) - m;
        float f3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7443)) - m;
        p01 = pack(f0, f1);
        p23 = pack(f2, f3);
    }
};

__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MinGRU cell (k_mingru_epi_fwd, craftax_full.cu:9377-9381) with
// sigmoid(z) = 0.5 + 0.5 tanh(z/2) on the SFU and g(z) - 0.5 = max(z, 0.5 tanh(z/2))
// (equal to z for z >= 0 and to sigmoid(z) - 0.5 for z < 0).
__device__ __forceinline__ void mingru_cell(float zh, float zg, float zp, float st, float x,
                                            float& out, float& h) {
    const float th = tanh_fast(0.5f * zh), tg = tanh_fast(0.5f * zg), tp = tanh_fast(0.5f * zp);
    const float sg = fmaf(tg, 0.5f, 0.5f), p = fmaf(tp, 0.5f, 0.5f);
    const float gh = 0.5f + fmaxf(zh, 0.5f * th);
    out = fmaf(sg, gh - st, st);
    h = fmaf(p, out - x, x);
}

struct Smem {
    uint8_t* base;
    __device__ __forceinline__ uint32_t bar(int i) const { return smem_u32(base + kOffBars + i * 8); }
    __device__ __forceinline__ uint8_t* b_slot(int s) const { return base + kOffB + s * kBSlot; }
    __device__ __forceinline__ uint8_t* s_slot(int s) const { return base + kOffS + s * kSSlot; }
    __device__ __forceinline__ uint8_t* r_slot(int s) const { return base + kOffR + s * kRSlot; }
    __device__ __forceinline__ float* bias() const { return reinterpret_cast<float*>(base + kOffBias); }
    __device__ __forceinline__ uint32_t* tmem_base() const { return reinterpret_cast<uint32_t*>(base + kOffMisc); }
    __device__ __forceinline__ volatile uint32_t* abort_flag() const {
        return reinterpret_cast<volatile uint32_t*>(base + kOffMisc + 4);
    }
};

// every role runs in its own function: a failed (timed-out) wait returns to the common exit
#define CFX_WAIT(barid, parity, code) \
    if (!mbar_wait(sm.bar(barid), (parity), sm.abort_flag(), (code))) return

// ------------------------------------------------------------------ producer roles
// Weight stages: the image is laid out in consumption order, so the source pointer just
// advances; every tile replays the same sequence (it stays L2 resident).
__device__ __forceinline__ void role_weight_loads(const Smem& sm, const Params& P) {
    const int stages_gate = P.L * kSlices * kKBlocks;
    uint32_t cnt = 0;
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x) {
        const uint8_t* src = P.image;
        for (int s = 0; s < kEncStages + stages_gate + kKBlocks; s++, cnt++) {
            const uint32_t bytes = s < kEncStages ? kEncStageBytes
                                   : (s < kEncStages + stages_gate ? kGateStageBytes : kHeadStageBytes);
            const int slot = cnt % kNB;
            CFX_WAIT(B_EMPTY + slot, ((cnt / kNB) & 1) ^ 1, W_B_EMPTY);
            mbar_arrive_expect_tx(sm.bar(B_FULL + slot), bytes);
            bulk_g2s(smem_u32(sm.b_slot(slot)), src, bytes, sm.bar(B_FULL + slot));
            src += bytes;
        }
    }
}

// Records: the [n][996] byte array is viewed as [n/4][3984] (four records per 16-byte
// aligned row); env 4g+i of a tile sits in row g at byte 996 i.  A 64-byte feature chunk of
// all 128 envs is fetched as four boxes (one per i) of 32 rows x 80 bytes starting at the
// 16-byte boundary below 996 i + 64 c; the 204 tail bytes take three more such box sets.
__device__ __forceinline__ void role_record_loads(const Smem& sm, const Params& P) {
    uint32_t cnt = 0;
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x) {
        for (int sub = 0; sub < kRecSubs; sub++, cnt++) {
            const int slot = cnt % kNR;
            CFX_WAIT(R_EMPTY + slot, ((cnt / kNR) & 1) ^ 1, W_R_EMPTY);
            mbar_arrive_expect_tx(sm.bar(R_FULL + slot), kRSlot);
            const int byte0 = sub < 13 ? 64 * sub : kMap + 80 * (sub - 13);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int x0 = sub < 13 ? ((kRec * i + byte0) & ~15)
                                        : ((kRec * i + kMap) & ~15) + 80 * (sub - 13);
                tensor_g2s_2d(smem_u32(sm.r_slot(slot) + i * kRBoxBytes), &P.rec_map, x0, tile * 32,
                              sm.bar(R_FULL + slot));
            }
        }
    }
}

// State slices: layer l, tile rows, 32 units -> one 16 KB box, 128-byte swizzled.
__device__ __forceinline__ void role_state_loads(const Smem& sm, const Params& P) {
    uint32_t cnt = 0;
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x) {
        for (int l = 0; l < P.L; l++) {
            for (int j = 0; j < kSlices; j++, cnt++) {
                const int slot = cnt % kNS;
                CFX_WAIT(S_EMPTY + slot, ((cnt / kNS) & 1) ^ 1, W_S_EMPTY);
                mbar_arrive_expect_tx(sm.bar(S_FULL + slot), kSSlot);
                tensor_g2s_2d(smem_u32(sm.s_slot(slot)), &P.state_map[l], j * kSliceUnits,
                              tile * kTile, sm.bar(S_FULL + slot));
            }
        }
    }
}

// The workers overwrite a state slot in place with the new state; this warp writes it
// back (rows beyond n are clipped by the tensor map) and recycles the slot.
__device__ __forceinline__ void role_state_stores(const Smem& sm, const Params& P) {
    uint32_t cnt = 0;
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x) {
        for (int l = 0; l < P.L; l++) {
            for (int j = 0; j < kSlices; j++, cnt++) {
                const int slot = cnt % kNS;
                CFX_WAIT(ST_READY + slot, (cnt / kNS) & 1, W_ST_READY);
                tensor_s2g_2d(&P.state_map[l], smem_u32(sm.s_slot(slot)), j * kSliceUnits,
                              tile * kTile);
                bulk_commit_group();
                bulk_wait_group_read<0>();
                mbar_arrive(sm.bar(S_EMPTY + slot));
            }
        }
    }
}

// ------------------------------------------------------------------ MMA role
template <typename T16>
__device__ __forceinline__ void role_mma(const Smem& sm, const Params& P, uint32_t tmem) {
    constexpr uint32_t fmt = Op16<T16>::kFmt;
    constexpr uint32_t idesc_enc = make_idesc(fmt, 128, 128);
    constexpr uint32_t idesc_gate = make_idesc(fmt, 128, 3 * kSliceUnits);
    constexpr uint32_t idesc_head = make_idesc(fmt, 128, kHeadN);
    uint32_t bcnt = 0, acnt = 0, akb_use = 0, gcnt[2] = {0, 0};
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x) {
        // ---- encoder: 14 operand chunks x 2 unit halves
        for (int kc = 0; kc < kEncChunks; kc++, acnt++) {
            const int as = acnt % kAexpSlots;
            CFX_WAIT(AEXP_FULL + as, (acnt / kAexpSlots) & 1, W_AEXP_FULL);
            tc_fence_after_sync();
            const int ksteps = kc == 12 ? 2 : 4;
            const uint32_t a_col = tmem + kColAexp + as * 32;
            for (int half = 0; half < 2; half++, bcnt++) {
                const int slot = bcnt % kNB;
                CFX_WAIT(B_FULL + slot, (bcnt / kNB) & 1, W_B_FULL);
                tc_fence_after_sync();
                const uint32_t b_addr = smem_u32(sm.b_slot(slot));
                for (int ks = 0; ks < ksteps; ks++)
                    mma_f16_ts(tmem + kColAcc + half * 128, a_col + ks * 8,
                               smem_desc_sw128(b_addr + ks * 32), idesc_enc, (kc | ks) != 0);
                mma_commit(sm.bar(B_EMPTY + slot));
            }
            mma_commit(sm.bar(AEXP_EMPTY + as));
        }
        mma_commit(sm.bar(ACC_FULL));
        // ---- MinGRU layers: 8 slices x 4 K blocks, N = 96 (zh|zg|zp of 32 units)
        for (int l = 0; l < P.L; l++, akb_use++) {
            const uint32_t a_cur = tmem + ((l & 1) ? kColA1 : kColA0);
            for (int j = 0; j < kSlices; j++) {
                const int g = j & 1;
                CFX_WAIT(G_EMPTY + g, (gcnt[g] & 1) ^ 1, W_G_EMPTY);
                gcnt[g]++;
                tc_fence_after_sync();
                const uint32_t d_col = tmem + (g ? kColG1 : kColG0);
                for (int kb = 0; kb < kKBlocks; kb++, bcnt++) {
                    if (j == 0) {
                        CFX_WAIT(A_KB + kb, akb_use & 1, W_A_KB);
                        tc_fence_after_sync();
                    }
                    const int slot = bcnt % kNB;
                    CFX_WAIT(B_FULL + slot, (bcnt / kNB) & 1, W_B_FULL);
                    tc_fence_after_sync();
                    const uint32_t b_addr = smem_u32(sm.b_slot(slot));
                    for (int ks = 0; ks < 4; ks++)
                        mma_f16_ts(d_col, a_cur + kb * 32 + ks * 8, smem_desc_sw128(b_addr + ks * 32),
                                   idesc_gate, (kb | ks) != 0);
                    mma_commit(sm.bar(B_EMPTY + slot));
                }
                mma_commit(sm.bar(G_FULL + g));
            }
        }
        // ---- heads: N = 48
        {
            const uint32_t a_cur = tmem + ((P.L & 1) ? kColA1 : kColA0);
            for (int kb = 0; kb < kKBlocks; kb++, bcnt++) {
                CFX_WAIT(A_KB + kb, akb_use & 1, W_A_KB);
                tc_fence_after_sync();
                const int slot = bcnt % kNB;
                CFX_WAIT(B_FULL + slot, (bcnt / kNB) & 1, W_B_FULL);
                tc_fence_after_sync();
                const uint32_t b_addr = smem_u32(sm.b_slot(slot));
                for (int ks = 0; ks < 4; ks++)
                    mma_f16_ts(tmem + kColHead, a_cur + kb * 32 + ks * 8,
                               smem_desc_sw128(b_addr + ks * 32), idesc_head, (kb | ks) != 0);
                mma_commit(sm.bar(B_EMPTY + slot));
            }
            akb_use++;
            mma_commit(sm.bar(H_FULL));
        }
    }
}

// ------------------------------------------------------------------ worker role
// Eight warps, two per TMEM lane quarter (wg 0 / wg 1); thread (quarter, lane) owns env row
// quarter*32 + lane of the tile in every phase.
template <typename T16>
__device__ __forceinline__ void role_worker(const Smem& sm, const Params& P, uint32_t tmem,
                                            int warp, int lane) {
    using Op = Op16<T16>;
    const int wg = (warp - kWorkerWarp0) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int gi = row >> 2, ii = row & 3;
    const float* bias = sm.bias();
    const uint32_t rec_row_off = ii * kRBoxBytes + gi * 80;
    uint32_t rcnt = 0, acnt = 0, tcnt = 0, gcnt = 0, it = 0;
    for (int tile = blockIdx.x; tile < P.num_tiles; tile += gridDim.x, it++, tcnt++) {
        const int env = tile * kTile + row;
        const bool valid = env < P.n;
        const bool zero_state =
            valid && P.prev_terminals != nullptr && P.prev_terminals[env] != 0.0f;

        // ---- expand: record bytes -> 16-bit operand rows in the TMEM chunk ring
        for (int kc = 0; kc < kEncChunks; kc++, acnt++) {
            const int as = acnt % kAexpSlots;
            CFX_WAIT(AEXP_EMPTY + as, ((acnt / kAexpSlots) & 1) ^ 1, W_AEXP_EMPTY);
            tc_fence_after_sync();
            uint32_t regs[16];
            if (kc < 13) {
                const int slot = rcnt % kNR;
                CFX_WAIT(R_FULL + slot, (rcnt / kNR) & 1, W_R_FULL);
                const uint8_t* src = sm.r_slot(slot) + rec_row_off + ((kRec * ii) & 15) + 32 * wg;
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    uint32_t w32 = *reinterpret_cast<const uint32_t*>(src + 4 * q);
                    if (kc == 12 && (wg == 1 || q >= 6)) w32 = 0;  // bytes 792.. are not map bytes
                    Op::bytes4(w32, regs[2 * q], regs[2 * q + 1]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sm.bar(R_EMPTY + slot));
                rcnt++;
            } else {
#pragma unroll
                for (int s = 0; s < 3; s++)
                    CFX_WAIT(R_FULL + (rcnt + s) % kNR, ((rcnt + s) / kNR) & 1, W_R_FULL);
                const uint32_t rem = (kRec * ii + kMap) & 15;
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    float v[2];
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int f = 32 * wg + 2 * q + e;  // tail float index (wg is warp-uniform)
                        v[e] = 0.0f;
                        if (f < kTail) {
                            const uint32_t off = rem + 4 * f;
                            const uint32_t sidx = off / 80, within = off - sidx * 80;
                            v[e] = *reinterpret_cast<const float*>(
                                sm.r_slot((rcnt + sidx) % kNR) + rec_row_off + within);
                        }
                    }
                    regs[q] = Op::pack(v[0], v[1]);
                }
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (int s = 0; s < 3; s++) mbar_arrive(sm.bar(R_EMPTY + (rcnt + s) % kNR));
                }
                rcnt += 3;
            }
            tmem_st16(tmem + lane_base + kColAexp + as * 32 + 16 * wg, regs);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(sm.bar(AEXP_FULL + as));
        }

        // ---- encoder epilogue: accumulator + bias -> layer-0 input A0 (wg = unit half)
        CFX_WAIT(ACC_FULL, tcnt & 1, W_ACC_FULL);
        tc_fence_after_sync();
#pragma unroll 2
        for (int b = 0; b < 8; b++) {
            uint32_t acc[16], pk[8];
            tmem_ld16(tmem + lane_base + kColAcc + 128 * wg + 16 * b, acc);
            tmem_wait_ld();
            const float* bb = bias + 128 * wg + 16 * b;
#pragma unroll
            for (int q = 0; q < 8; q++)
                pk[q] = Op::pack(__uint_as_float(acc[2 * q]) + bb[2 * q],
                                 __uint_as_float(acc[2 * q + 1]) + bb[2 * q + 1]);
            tmem_st8(tmem + lane_base + kColA0 + 64 * wg + 8 * b, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(sm.bar(A_KB + 2 * wg));
            mbar_arrive(sm.bar(A_KB + 2 * wg));
            mbar_arrive(sm.bar(A_KB + 2 * wg + 1));
            mbar_arrive(sm.bar(A_KB + 2 * wg + 1));
        }

        // ---- MinGRU layers: wg handles slices j = wg, wg+2, ... from gate buffer G[wg]
        for (int l = 0; l < P.L; l++) {
            const uint32_t a_cur = tmem + lane_base + ((l & 1) ? kColA1 : kColA0);
            const uint32_t a_next = tmem + lane_base + ((l & 1) ? kColA0 : kColA1);
            for (int jj = 0; jj < kSlices / 2; jj++, gcnt++) {
                const int j = 2 * jj + wg;
                CFX_WAIT(G_FULL + wg, gcnt & 1, W_G_FULL);
                tc_fence_after_sync();
                const uint32_t scnt = (it * P.L + l) * kSlices + j;
                const int slot = scnt % kNS;
                const uint32_t gcol = tmem + lane_base + (wg ? kColG1 : kColG0);
                uint8_t* rbase = sm.s_slot(slot) + (row >> 3) * 1024 + (row & 7) * 128;
                const int xr = row & 7;
                bool state_ready = false;
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    uint32_t zh[16], zg[16], zp[16], xin[8], hn[8];
                    tmem_ld16(gcol + 16 * hf, zh);
                    tmem_ld16(gcol + 32 + 16 * hf, zg);
                    tmem_ld16(gcol + 64 + 16 * hf, zp);
                    tmem_ld8(a_cur + 16 * j + 8 * hf, xin);
                    tmem_wait_ld();
                    if (hf == 1) {  // all gate columns of this slice are in registers
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sm.bar(G_EMPTY + wg));
                    }
                    if (!state_ready) {
                        CFX_WAIT(S_FULL + slot, (scnt / kNS) & 1, W_S_FULL);
                        state_ready = true;
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        float4* sp = reinterpret_cast<float4*>(rbase + (((4 * hf + q) ^ xr) << 4));
                        float4 st = *sp;
                        if (zero_state) st = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float2 x01 = Op::unpack(xin[2 * q]), x23 = Op::unpack(xin[2 * q + 1]);
                        float4 out;
                        float h0, h1, h2, h3;
                        mingru_cell(__uint_as_float(zh[4 * q]), __uint_as_float(zg[4 * q]),
                                    __uint_as_float(zp[4 * q]), st.x, x01.x, out.x, h0);
                        mingru_cell(__uint_as_float(zh[4 * q + 1]), __uint_as_float(zg[4 * q + 1]),
                                    __uint_as_float(zp[4 * q + 1]), st.y, x01.y, out.y, h1);
                        mingru_cell(__uint_as_float(zh[4 * q + 2]), __uint_as_float(zg[4 * q + 2]),
                                    __uint_as_float(zp[4 * q + 2]), st.z, x23.x, out.z, h2);
                        mingru_cell(__uint_as_float(zh[4 * q + 3]), __uint_as_float(zg[4 * q + 3]),
                                    __uint_as_float(zp[4 * q + 3]), st.w, x23.y, out.w, h3);
                        *sp = out;
                        hn[2 * q] = Op::pack(h0, h1);
                        hn[2 * q + 1] = Op::pack(h2, h3);
                    }
                    tmem_st8(a_next + 16 * j + 8 * hf, hn);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sm.bar(A_KB + (j >> 1)));
                    mbar_arrive(sm.bar(ST_READY + slot));
                }
            }
        }

        // ---- heads + sampler (wg 0: one thread per env; wg 1 only passes the barrier so
        // that its next-tile operand writes cannot overtake the last MMA)
        CFX_WAIT(H_FULL, tcnt & 1, W_H_FULL);
        tc_fence_after_sync();
        if (wg == 0) {
            uint32_t hv[kHeadN];
#pragma unroll
            for (int b = 0; b < kHeadN / 16; b++) {
                uint32_t t[16];
                tmem_ld16(tmem + lane_base + kColHead + 16 * b, t);
#pragma unroll
                for (int q = 0; q < 16; q++) hv[16 * b + q] = t[q];
            }
            tmem_wait_ld();
            tc_fence_before_sync();
            if (valid) {
                float logits[kA];
#pragma unroll
                for (int a = 0; a < kA; a++) logits[a] = __uint_as_float(hv[a]) + bias[kH + a];
                const float value = __uint_as_float(hv[kA]) + bias[kH + kA];
                if (P.logits_av != nullptr) {
                    float4* dst = reinterpret_cast<float4*>(P.logits_av + (size_t)env * (kA + 1));
#pragma unroll
                    for (int q = 0; q < (kA + 1) / 4; q++) {
                        float4 v4;
                        v4.x = logits[4 * q];
                        v4.y = logits[4 * q + 1];
                        v4.z = logits[4 * q + 2];
                        v4.w = (4 * q + 3 < kA) ? logits[(4 * q + 3 < kA) ? 4 * q + 3 : 0] : value;
                        dst[q] = v4;
                    }
                }
                const float u = P.uniforms != nullptr
                                    ? P.uniforms[env]
                                    : philox_uniform(P.seed, P.env_offset + (uint64_t)env, *P.step_ctr);
                float lp;
                const int act = sample_action<kA>(logits, u, &lp);
                if (P.env_actions) P.env_actions[env] = (float)act;
                P.actions[env] = act;
                if (P.logprobs) P.logprobs[env] = lp;
                if (P.values) P.values[env] = value;
            }
        }
    }
}

// ------------------------------------------------------------------ kernel
template <typename T16>
__global__ void __launch_bounds__(kThreads, 1)
k_policy_fused(const __grid_constant__ Params P) {
    extern __shared__ uint8_t smem_raw[];
    Smem sm;
    sm.base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        auto init = [&](int first, int count, uint32_t arrivals) {
            for (int i = 0; i < count; i++) mbar_init(sm.bar(first + i), arrivals);
        };
        init(B_FULL, kNB, 1);
        init(B_EMPTY, kNB, 1);
        init(S_FULL, kNS, 1);
        init(S_EMPTY, kNS, 1);
        init(ST_READY, kNS, 4);
        init(R_FULL, kNR, 1);
        init(R_EMPTY, kNR, 8);
        init(AEXP_FULL, kAexpSlots, 8);
        init(AEXP_EMPTY, kAexpSlots, 1);
        init(ACC_FULL, 1, 1);
        init(A_KB, kKBlocks, 8);
        init(G_FULL, 2, 1);
        init(G_EMPTY, 2, 4);
        init(H_FULL, 1, 1);
        *sm.abort_flag() = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(sm.tmem_base()), 512);
        tmem_relinquish();
    }
    if (warp == 2 && lane == 0) {
        prefetch_tensormap(&P.rec_map);
        for (int l = 0; l < P.L; l++) prefetch_tensormap(&P.state_map[l]);
    }
    for (int i = tid; i < kH + kHeadN; i += kThreads) {
        float v = 0.0f;
        if (i < kH) v = P.params[P.off_b_enc + i];
        else if (i - kH < kA) v = P.params[P.off_b_a + (i - kH)];
        else if (i - kH == kA) v = P.params[P.off_b_v];
        sm.bias()[i] = v;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *sm.tmem_base();

    if (warp == 0) {
        if (lane == 0) role_weight_loads(sm, P);
    } else if (warp == 1) {
        if (lane == 0) role_mma<T16>(sm, P, tmem);
    } else if (warp == 2) {
        if (lane == 0) role_record_loads(sm, P);
    } else if (warp == 3) {
        if (lane == 0) role_state_loads(sm, P);
    } else if (warp == 4) {
        if (lane == 0) {
            role_state_stores(sm, P);
            bulk_wait_group<0>();
        }
    } else {
        role_worker<T16>(sm, P, tmem, warp, lane);
    }

    // common exit: every role ends here, also after a timed-out wait
    __syncwarp();
    tc_fence_before_sync();
    __syncthreads();
    const uint32_t aborted = *sm.abort_flag();
    if (aborted != 0) {
        if (tid == 0) atomicCAS(P.status, 0u, aborted | ((uint32_t)blockIdx.x << 8));
        // give copies that are still in flight time to land before shared memory is released
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace fused

// ------------------------------------------------------------------ host side
struct FusedPlan {
    int device, n, H, L, A, precision;
    uint8_t* image = nullptr;
    uint32_t* status = nullptr;
    float* state = nullptr;
    const float* params = nullptr;
    CUtensorMap state_map[fused::kMaxLayers];
    int sm_count = 0;
};

bool fused_supported(int H, int L, int A, int precision) {
    return H == fused::kH && A == fused::kA && L >= 1 && L <= fused::kMaxLayers &&
           (precision == CFX_PREC_F16 || precision == CFX_PREC_BF16);
}

int fused_create(FusedPlan** out, int device, int n, int H, int L, int A, int precision,
                 float* state) {
    if (!fused_supported(H, L, A, precision)) {
        set_error("fused kernel: unsupported shape/precision");
        return CFX_ERR_UNSUPPORTED;
    }
    cudaDeviceProp prop;
    CFX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("fused kernel needs an sm_100 GPU (found sm_%d%d)", prop.major, prop.minor);
        return CFX_ERR_UNSUPPORTED;
    }
    FusedPlan* p = new FusedPlan();
    p->device = device; p->n = n; p->H = H; p->L = L; p->A = A; p->precision = precision;
    p->state = state;
    p->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaMalloc((void**)&p->image, fused::image_bytes(L));
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->status, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(p->status, 0, sizeof(uint32_t));
    if (e != cudaSuccess) {
        fused_destroy(p);
        return cuda_fail(e, "fused_create alloc", __FILE__, __LINE__);
    }
    for (int l = 0; l < L; l++) {
        if (!make_tmap_2d(&p->state_map[l], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                          state + (size_t)l * n * H, (uint64_t)n, (uint64_t)H, (uint64_t)H * 4,
                          fused::kTile, fused::kSliceUnits, CU_TENSOR_MAP_SWIZZLE_128B)) {
            fused_destroy(p);
            set_error("fused_create: cuTensorMapEncodeTiled failed for the state");
            return CFX_ERR_CUDA;
        }
    }
    e = cudaFuncSetAttribute(fused::k_policy_fused<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fused::kSmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(fused::k_policy_fused<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, fused::kSmemBytes);
    if (e != cudaSuccess) {
        fused_destroy(p);
        return cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__);
    }
    *out = p;
    return CFX_OK;
}

int fused_refresh(FusedPlan* p, const float* params, cudaStream_t st) {
    p->params = params;
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A);
    const size_t total = fused::image_bytes(p->L) / 2;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (p->precision == CFX_PREC_F16)
        fused::k_pack_image<__half><<<blocks, 256, 0, st>>>(params, p->image, p->L, o.w_gru, o.w_a, o.w_v);
    else
        fused::k_pack_image<__nv_bfloat16><<<blocks, 256, 0, st>>>(params, p->image, p->L, o.w_gru, o.w_a, o.w_v);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int fused_forward(FusedPlan* p, const FusedArgs& a, cudaStream_t st, int* launches) {
    if (a.r_state != nullptr) {
        set_error("fused forward: r_state recording is only available with precision fp32");
        return CFX_ERR_UNSUPPORTED;
    }
    if (a.logits_av != nullptr && ((uintptr_t)a.logits_av & 15) != 0) {
        set_error("fused forward: logits_av must be 16-byte aligned");
        return CFX_ERR_INVALID;
    }
    fused::Params P;
    if (!make_tmap_2d(&P.rec_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (void*)a.records,
                      (uint64_t)p->n / 4, (uint64_t)kRec * 4, (uint64_t)kRec * 4, 32, 80,
                      CU_TENSOR_MAP_SWIZZLE_NONE)) {
        set_error("fused forward: cuTensorMapEncodeTiled failed for the records");
        return CFX_ERR_CUDA;
    }
    for (int l = 0; l < p->L; l++) P.state_map[l] = p->state_map[l];
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A);
    P.image = p->image;
    P.params = p->params;
    P.prev_terminals = a.prev_terminals;
    P.uniforms = a.uniforms;
    P.env_actions = a.env_actions;
    P.actions = a.actions;
    P.logprobs = a.logprobs;
    P.values = a.values;
    P.logits_av = a.logits_av;
    P.step_ctr = a.step_ctr;
    P.status = p->status;
    P.seed = a.seed;
    P.env_offset = a.env_offset;
    P.n = p->n;
    P.L = p->L;
    P.num_tiles = (p->n + fused::kTile - 1) / fused::kTile;
    P.off_b_enc = o.b_enc;
    P.off_b_a = o.b_a;
    P.off_b_v = o.b_v;
    const int grid = P.num_tiles < p->sm_count ? P.num_tiles : p->sm_count;
    if (p->precision == CFX_PREC_F16)
        fused::k_policy_fused<__half><<<grid, fused::kThreads, fused::kSmemBytes, st>>>(P);
    else
        fused::k_policy_fused<__nv_bfloat16><<<grid, fused::kThreads, fused::kSmemBytes, st>>>(P);
    CFX_CUDA(cudaGetLastError());
    if (launches) *launches = 1;
    return CFX_OK;
}

int fused_check_status(FusedPlan* p, cudaStream_t st, unsigned* status) {
    uint32_t v = 0;
    CFX_CUDA(cudaMemcpyAsync(&v, p->status, sizeof(v), cudaMemcpyDeviceToHost, st));
    CFX_CUDA(cudaStreamSynchronize(st));
    if (v != 0) CFX_CUDA(cudaMemsetAsync(p->status, 0, sizeof(v), st));
    if (status) *status = v;
    return CFX_OK;
}

void fused_destroy(FusedPlan* p) {
    if (!p) return;
    if (p->image) cudaFree(p->image);
    if (p->status) cudaFree(p->status);
    delete p;
}

}  // namespace cfx
