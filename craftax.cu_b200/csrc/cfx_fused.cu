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
// Tile-level dataflow (M = 128 envs = the 128 TMEM lanes; the worker thread that owns TMEM lane
// r owns env row r of the tile in every phase):
//   TMEM columns   gate phase: A0 [0,128) A1 [128,256) (layer inputs, 16-bit packed, ping-pong)
//                              G [256,448) (gate accumulators of one 64-unit slice: zh|zg|zp;
//                              the workers move it to registers at once, which frees it for
//                              the next slice's MMAs while the cell runs)  HEAD [448,512)
//                  encoder phase: operand-chunk ring [0,256) (8 x 32 columns), accumulator
//                              [256,512)
//   shared memory  weight ring | state ring (four of the six record slots live inside its slots)
//                  | two record slots / classic record buffer | biases, barriers: see Cfg
//   warps          0 weight loads, 1 MMA issue + TMEM alloc, 2 record fills of worker warpgroup 1
//                  + state box loads + the L2 prefetch, 3 record fills of warpgroup 0 + state
//                  box stores (one thread each), 4..11 workers (expand, cell, sampler)
//   launch modes   clusters of two CTAs sharing 256-row MMAs (PAIR, the default) or one CTA per
//                  tile; full game or classic game (GAME): see Cfg and Gm
//   hidden size    256 (the figures in this comment) or 128 (HID): two gate slices of two K
//                  blocks per layer, A0 / A1 of 64 columns, encoder accumulator N = 128: see Hd
// One round of (mbarrier wait, arrive.expect_tx, bulk copy) costs its issuing thread about
// 500 cycles on B200.  Every copy role is ONE thread that walks its ring in order: the slots of
// a ring come free in the order they were filled, and several lanes of one warp, each in its own
// loop, serve their slots far more slowly than one thread serves them all.
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

constexpr int kTile = 128;       // envs per tile
constexpr int kMaxLayers = 4;
constexpr int kSliceUnits = 64;  // hidden units per gate slice (N = 192: zh|zg|zp)
constexpr int kHalfUnits = 32;   // units of a slice handled by one worker warpgroup
constexpr int kHeadMax = 64;     // head accumulator columns reserved in tensor memory
// Shapes that follow from the hidden size the kernel is instantiated for (256 or 128).
template <int HID> struct Hd {
    static_assert(HID == 256 || HID == 128, "hidden sizes the kernel is built for");
    static constexpr int kH = HID;                        // hidden units
    static constexpr int kSlices = HID / kSliceUnits;     // gate slices per layer (4 / 2)
    static constexpr int kStateItems = HID / kHalfUnits;  // state boxes (128 rows x 32 units) per layer (8 / 4)
    static constexpr int kKBlocks = HID / 64;             // K blocks of 64 per HID-wide operand (4 / 2)
    static constexpr int kEncBlockBytes = HID * 128;      // one encoder chunk: [HID units][64 K] 16-bit
    static constexpr int kEncCopyBytes = 2 * HID * 128;   // encoder stage: two chunks
    static_assert((HID / 64) % 2 == 0, "a gate stage carries two K blocks");
};
// brings the shapes of Hd<HID> into a function body
#define CFX_DIMS(HID)                                                                        \
    constexpr int kH = Hd<HID>::kH, kSlices = Hd<HID>::kSlices, kStateItems = Hd<HID>::kStateItems, \
                  kKBlocks = Hd<HID>::kKBlocks, kEncCopyBytes = Hd<HID>::kEncCopyBytes;      \
    (void)kH; (void)kSlices; (void)kStateItems; (void)kKBlocks; (void)kEncCopyBytes

// What differs between the two games the kernel is instantiated for.
//  full game (craftax_full.cu): 996-byte record = 792 map bytes + 51 raw floats, 843 features.
//    The record goes through the record ring in 16 chunks of 64 RECORD bytes: chunks 0-11 are 64
//    map bytes each (four K steps), chunk 12 is 24 map bytes and floats 0-9 (three K steps),
//    chunks 13 and 14 are 16 floats each and chunk 15 the last 9 floats (one K step each).  The
//    weight image has 14 blocks of 64 K columns: blocks 0-11 belong to chunks 0-11, block 12 to
//    chunks 12 and 13 (K columns 0-47 and 48-63), block 13 to chunks 14 and 15 (K columns 0-15
//    and 16-31).  43 actions;
//  classic game (craftax_classic.cu): 148-byte record, 1345 one-hot / scalar features in 22
//    chunks (one weight block each), the whole tile's records (18.5 KB) fetched by one TMA box,
//    17 actions.
template <int GAME> struct Gm;
template <> struct Gm<CFX_GAME_FULL> {
    static constexpr int kA = 43, kEncChunks = 16, kEncBlocks = 14, kRecBytes = kRec;
    static constexpr int kHeadSingle = 48, kHeadPair = 64;   // head MMA N (pairs need N % 32 == 0)
};
template <> struct Gm<CFX_GAME_CLASSIC> {
    static constexpr int kA = 17, kEncChunks = 22, kEncBlocks = 22, kRecBytes = kClassicRec;
    static constexpr int kHeadSingle = 32, kHeadPair = 32;
};

constexpr int kNBMax = 8;        // weight ring slots (one stage each): see Cfg
// Ring shapes (measured at 262,144 envs, h256x2, CTA pairs: four weight slots with four state
// slots beat three weight slots with six state slots by 3 %, and six state slots with every
// record slot inside one of them lost 2.6 % against four state slots plus two record slots of
// their own: the weight ring's depth hides the L2 round trip of a stage, and the two record
// slots outside the state ring are filled for the next tile while the gate layers still run)
constexpr int kSSlot = 16384, kNSMax = 4;
constexpr int kRBoxBytes = 32 * 80, kRSlot = 4 * kRBoxBytes, kNRMax = 6;
constexpr int kOwnRSlots = 2;    // record slots outside the state slots (the classic record buffer's place)
constexpr int kAexpSlots = 8;
constexpr int kKBlocksMax = 4;

// Image blocks (one K block of 64 columns each) and the ring stages that carry them.  A stage
// holds TWO blocks, so that the MMA thread waits, probes and commits once per eight MMAs:
// encoder stage = two chunks of 256 units (2 x 32 KB); gate stage = two K blocks of one 64-unit
// slice (2 x 192 rows, 2 x 24 KB); head stage = all K blocks.  One CTA per tile stages whole
// stages, [block][rows][64 K]; in a CTA pair every CTA stages its half of the rows of both
// blocks, laid out [half][block][rows / 2][64 K] so that a CTA's part is one contiguous copy.
constexpr int kStageBlocks = 2;
constexpr int kGateBlockBytes = 3 * kSliceUnits * 128;               // block: [192 rows][64 K]
constexpr int kGateStageBytes = kStageBlocks * kGateBlockBytes;
// head stage: one CTA per tile [K block][rows][64 K]; pairs [half][K block][rows / 2][64 K]
template <int GAME, int HID> __host__ __device__ constexpr int head_bytes(bool pair) {
    return Hd<HID>::kKBlocks * (pair ? Gm<GAME>::kHeadPair : Gm<GAME>::kHeadSingle) * 128;
}
template <int GAME, int HID> __host__ __device__ constexpr size_t enc_bytes() {
    static_assert(Gm<GAME>::kEncBlocks % 2 == 0, "an encoder stage carries two blocks");
    return (size_t)Gm<GAME>::kEncBlocks * Hd<HID>::kEncBlockBytes;
}

// Barriers are waited on by phase parity, which is only sound while the waiter can never be
// two phases off.  So every slot of a ring has ONE filling thread and ONE consuming warpgroup
// for the whole launch (a consumer that skipped slots owned by others could be two phases
// off), and both keep the slot's phase as a running count of their own uses: the record ring
// (three slots per warpgroup), the state ring (4 slots, boxes alternate between the
// warpgroups), the weight ring (one consumer).  The operand slots in tensor memory are shared
// by the two warpgroups (chunk c and chunk c + 8 use the same slot); there the order is carried
// by the previous tile's H_FULL, which both have passed.

template <int GAME, int HID> __host__ __device__ constexpr size_t image_bytes(int L) {   // room for either head layout
    return enc_bytes<GAME, HID>() + (size_t)L * Hd<HID>::kSlices * Hd<HID>::kKBlocks * kGateBlockBytes +
           (size_t)Hd<HID>::kKBlocks * kHeadMax * 128;
}

// TMEM columns
constexpr uint32_t kColA0 = 0, kColA1 = 128, kColG = 256, kColHead = 448;
constexpr uint32_t kColAexp = 0, kColAcc = 256;

constexpr int kOwnBytes = kOwnRSlots * kRSlot;   // two record slots, or the classic tile's records
enum Bar {
    B_FULL = 0, B_EMPTY = B_FULL + kNBMax, S_FULL = B_EMPTY + kNBMax, S_FREE = S_FULL + kNSMax,
    ST_READY = S_FREE + kNSMax, R_FULL = ST_READY + kNSMax, R_EMPTY = R_FULL + kNRMax,
    AEXP_FULL = R_EMPTY + kNRMax, AEXP_EMPTY = AEXP_FULL + kAexpSlots,
    ACC_FULL = AEXP_EMPTY + kAexpSlots, A_KB = ACC_FULL + 1, G_FULL = A_KB + kKBlocksMax,
    G_EMPTY = G_FULL + 1, H_FULL = G_EMPTY + 1, H_EMPTY = H_FULL + 1, REC_DONE = H_EMPTY + 1,
    ACC_READ = REC_DONE + 1, T_FULL = ACC_READ + 1, T_EMPTY = T_FULL + 1, NUM_BARS = T_EMPTY + 1
};

// Shared memory map (offsets from a 1024-byte aligned base) and the shapes that depend on the
// launch mode.
//  one CTA per tile: weight ring 2 x 64 KB (whole two-block stages), state ring 4 x 16 KB;
//  CTA pair (cta_group::2): every CTA stages half of each weight stage, 4 x 32 KB, state ring
//    4 x 16 KB.
//  In both modes four of the six record slots (10 KB each) live INSIDE the state slots: records
//  are needed only while the encoder runs, state boxes only while the gate layers run; REC_DONE
//  and S_FREE order the two uses per tile.  The other two slots have room of their own, so the
//  first chunks of the next tile are fetched while the gate layers of this one still run.
template <bool PAIR, int GAME, int HID> struct Cfg {
    static constexpr int kH = HID, kStateItems = Hd<HID>::kStateItems;
    static constexpr int kNB = PAIR ? 4 : 2;             // stages of two blocks (128 KB of weights in flight)
    static constexpr int kBSlot = PAIR ? 32768 : 65536;
    static constexpr int kHeadRows = PAIR ? Gm<GAME>::kHeadPair : Gm<GAME>::kHeadSingle;   // N of the head MMA
    static constexpr int kHeadKbBytes = (PAIR ? kHeadRows / 2 : kHeadRows) * 128;   // one K block of the head rows a CTA stages
    static constexpr int kM = PAIR ? 256 : 128;
    // state ring slots: even, so that slot parity = warpgroup; at most one layer's boxes
    static constexpr int kNS = 4;
    // record ring inside the state slots (full game only: the classic records need no ring)
    static constexpr bool kAlias = GAME == CFX_GAME_FULL;
    static constexpr int kOwn = GAME == CFX_GAME_FULL ? kOwnRSlots : 0;   // record slots beside the state slots
    static constexpr int kNR = GAME != CFX_GAME_FULL ? 0 : kOwn + kNS;
    static constexpr int kOffB = 0;
    static constexpr int kOffS = kOffB + kNB * kBSlot;
    static constexpr int kOffT = kOffS + kNS * kSSlot;         // own record slots / classic records
    static constexpr int kOffBias = kOffT + kOwnBytes;         // b_enc[256] fp32, b_av[48] fp32
    static constexpr int kOffBars = kOffBias + (kH + kHeadMax) * 4;
    static constexpr int kOffMisc = kOffBars + NUM_BARS * 8;  // tmem base, abort flag
    static constexpr int kSmemBytes = kOffMisc + 16 + 1024;   // + alignment slack
    static_assert(kNB <= kNBMax && kNR <= kNRMax && kNS <= kNSMax && kNS % 2 == 0 && kNS <= kStateItems &&
                      kRSlot <= kSSlot && kSmemBytes <= 232448 && kNS == 4 &&
                      kHeadRows <= kHeadMax && 128 * kClassicRec <= kOwnBytes, "layout");
};

constexpr int kWorkerWarp0 = 4, kNumWarps = 12, kThreads = kNumWarps * 32;

// wait-site codes recorded in the status word when a bounded wait gives up
enum WaitCode : uint32_t {
    W_B_EMPTY = 1, W_B_FULL, W_R_EMPTY, W_R_FULL, W_S_EMPTY, W_S_FULL, W_ST_READY, W_AEXP_EMPTY,
    W_AEXP_FULL, W_ACC_FULL, W_A_KB, W_G_FULL, W_G_EMPTY, W_H_FULL, W_H_EMPTY, W_REC_DONE, W_S_FREE, W_T_FULL, W_T_EMPTY, W_ACC_READ
};

struct Params {
    CUtensorMap rec_map;                 // uint8 [n/4][3984], box 32 x 80
    // pair mode: the operand image as [rows][64] 16-bit tensors, one map per region (encoder,
    // gate layers, heads); a box is the part of a stage that one CTA of the pair copies
    CUtensorMap w_map[3];
    CUtensorMap state_map[kMaxLayers];   // fp32 [n][256] per layer, box 128 x 32, SWIZZLE_128B
    const uint8_t* records;              // [n][996], for the L2 prefetch of the next tile
    const float* state;                  // [L][n][256]
    const uint8_t* image;                // pre-swizzled 16-bit weight stages in consumption order
    const float* params;                 // fp32 arena (biases are read from it)
    const float* prev_terminals;
    const float* uniforms;
    float* env_actions;
    int32_t* actions;
    float* logprobs;
    float* values;
    float* logits_av;
    float* r_state;                      // optional [L][n][H] record of the post-zero input state
    int r_state_bf16;                    // the record holds bf16 instead of fp32
    unsigned long long* step_ctr;        // device step counter (Philox offset); see bump_step
    uint32_t* status;
    uint32_t* done_ctr;                  // blocks that have finished this launch (bump_step)
    int bump_step;
    uint64_t seed, env_offset;
    int n, L, num_tiles;  // num_tiles: end of the tile range of this launch (exclusive)
    int tile_begin;       // first tile of this launch (a launch may cover a slice of the envs)
    int rec_bytes;        // bytes of one record (996 full game, 148 classic)
    int num_tiles_loop;   // trip bound of the tile loops: num_tiles, rounded up to even for CTA pairs
    size_t off_b_enc, off_b_a, off_b_v;
};

// ------------------------------------------------------------------ weight image
// Byte offset of (row, 16-bit K column c in [0,64)) inside a 128-byte-swizzled stage.
__host__ __device__ inline uint32_t sw128_off(uint32_t row, uint32_t byte_col) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((((byte_col >> 4) ^ (row & 7)) & 7) << 4) +
           (byte_col & 15);
}

// Feature behind K column c of encoder weight block `blk`, or -1 for padding.  Full game
// (feature kMap + i is raw float i of the record): blocks 0-11 map bytes 64 blk + c; block 12
// = map bytes 768-791, floats 0-9, 14 zero columns, floats 10-25; block 13 = floats 26-41,
// floats 42-50, zero columns.
template <int GAME> __host__ __device__ inline int enc_feature(int blk, int c) {
    if (GAME == CFX_GAME_CLASSIC) return blk * 64 + c < kClassicObs ? blk * 64 + c : -1;
    if (blk < 12) return blk * 64 + c;
    if (blk == 12) return c < 24 ? 768 + c : (c < 34 ? kMap + (c - 24) : (c < 48 ? -1 : kMap + 10 + (c - 48)));
    return c < 16 ? kMap + 26 + c : (c < 25 ? kMap + 42 + (c - 16) : -1);
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

// Position of one 16-bit element inside a two-block stage of `rows` rows per block: which
// block, which row of the block, which K column, and the byte offset of the element in the
// stage's shared-memory image (128-byte swizzled tiles).  `b` is the element's index-order byte
// offset in the stage; the mapping is a bijection of the stage's bytes.
struct StagePos { int blk, row, c; uint32_t dst; };
__host__ __device__ inline StagePos stage_pos(uint32_t b, int rows, bool pair) {
    StagePos p;
    if (pair) {   // [half][block][rows / 2][64 K]
        const uint32_t tile = (uint32_t)(rows / 2) * 128, half_bytes = kStageBlocks * tile;
        const uint32_t half = b / half_bytes, r2 = b % half_bytes, e = (r2 % tile) / 2;
        p.blk = (int)(r2 / tile);
        p.c = (int)(e % 64);
        p.row = (int)(half * (rows / 2) + e / 64);
        p.dst = half * half_bytes + (uint32_t)p.blk * tile + sw128_off(e / 64, (e % 64) * 2);
    } else {      // [block][rows][64 K]
        const uint32_t tile = (uint32_t)rows * 128, e = (b % tile) / 2;
        p.blk = (int)(b / tile);
        p.c = (int)(e % 64);
        p.row = (int)(e / 64);
        p.dst = (uint32_t)p.blk * tile + sw128_off(e / 64, (e % 64) * 2);
    }
    return p;
}

// One thread per 16-bit element of the image.  Stage order = consumption order of the
// kernel: encoder (chunk pairs), gate layers (layer, slice, K-block pair), head.
template <typename T16, int GAME, int HID>
__global__ void k_pack_image(const float* __restrict__ params, uint8_t* __restrict__ image, int L,
                             size_t off_w_gru, size_t off_w_a, size_t off_w_v, int pair) {
    CFX_DIMS(HID);
    constexpr int kA = Gm<GAME>::kA;
    const size_t total = image_bytes<GAME, HID>(L) / 2;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    size_t byte = idx * 2;
    const size_t enc_b = enc_bytes<GAME, HID>();
    const size_t gate_bytes = (size_t)L * kSlices * kKBlocks * kGateBlockBytes;
    float v = 0.0f;
    uint32_t row, c;
    uint8_t* stage;
    if (byte < enc_b) {
        const int s = (int)(byte / kEncCopyBytes);
        const StagePos q = stage_pos((uint32_t)(byte % kEncCopyBytes), kH, pair != 0);
        const int f = enc_feature<GAME>(kStageBlocks * s + q.blk, q.c);
        if (f >= 0) v = params[(size_t)f * kH + q.row];
        *reinterpret_cast<T16*>(image + (size_t)s * kEncCopyBytes + q.dst) = to16<T16>(v);
        return;
    } else if (byte < enc_b + gate_bytes) {
        const size_t b = byte - enc_b;
        const int s = (int)(b / kGateStageBytes);
        const StagePos q = stage_pos((uint32_t)(b % kGateStageBytes), 3 * kSliceUnits, pair != 0);
        constexpr int kPairsPerSlice = kKBlocks / kStageBlocks;
        const int kb = kStageBlocks * (s % kPairsPerSlice) + q.blk, j = (s / kPairsPerSlice) % kSlices,
                  l = s / (kPairsPerSlice * kSlices);
        const int gate = q.row / kSliceUnits, unit = j * kSliceUnits + q.row % kSliceUnits;
        // gate weights are stored halved: the accumulator then holds z / 2, the argument of the
        // cell's tanh (a power-of-two scale is exact for every weight above the subnormal range)
        v = 0.5f * params[off_w_gru + ((size_t)l * 3 * kH + gate * kH + unit) * kH + kb * 64 + q.c];
        *reinterpret_cast<T16*>(image + enc_b + (size_t)s * kGateStageBytes + q.dst) = to16<T16>(v);
        return;
    } else {
        // head.  One CTA per tile: [K block][rows][64 K].  CTA pairs: CTA r stages head rows
        // [r rows/2, (r + 1) rows/2): [r][K block][rows / 2][64 K].
        const size_t b = byte - enc_b - gate_bytes;
        if (b >= (size_t)head_bytes<GAME, HID>(pair != 0)) return;
        const int rows = pair ? Gm<GAME>::kHeadPair / 2 : Gm<GAME>::kHeadSingle;   // rows of one block
        const int blk_bytes = rows * 128;
        const int blk = (int)(b / blk_bytes), e = (int)((b % blk_bytes) / 2);
        const int r = pair ? blk / kKBlocks : 0, kb = blk % kKBlocks;
        row = e / 64; c = e % 64;
        stage = image + enc_b + gate_bytes + (size_t)blk * blk_bytes;
        const int grow = rows * r + (int)row;
        if (grow < kA) v = params[off_w_a + (size_t)grow * kH + kb * 64 + c];
        else if (grow == kA) v = params[off_w_v + kb * 64 + c];
    }
    *reinterpret_cast<T16*>(stage + sw128_off(row, c * 2)) = to16<T16>(v);
}

// ------------------------------------------------------------------ small device helpers
template <typename T16>
struct Op16;
template <>
struct Op16<__half> {
    static constexpr uint32_t kFmt = kFmtF16;
    static constexpr uint32_t kOne = 0x3C00u;   // 1.0
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
    static constexpr uint32_t kOne = 0x3F80u;   // 1.0
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

// MinGRU cell (k_mingru_epi_fwd, craftax_full.cu:9377-9381) with
// sigmoid(z) = 0.5 + 0.5 tanh(z/2) on the SFU and g(z) - 0.5 = max(z, 0.5 tanh(z/2))
// (equal to z for z >= 0 and to sigmoid(z) - 0.5 for z < 0).  The arguments are the HALVED
// pre-activations zh/2, zg/2, zp/2, which is what the gate MMAs produce (the operand image
// holds the gate weights times 0.5), so the cell starts with the tanh.
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two units at once with the packed fp32 instructions of sm_100 (`fma.rn.f32x2` and friends:
// two results per issue slot, the same roundings as the scalar forms).  The cell phase is
// bound by instruction issue and latency (two worker warps per scheduler), not by the FMA pipe.
__device__ __forceinline__ uint64_t f2pack(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2unpack(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2sub(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// hzh, hzg, hzp: zh/2, zg/2, zp/2 of two units
__device__ __forceinline__ void mingru_cell_pair(float hzh0, float hzh1, float hzg0, float hzg1, float hzp0,
                                                 float hzp1, float st0, float st1, float x0, float x1,
                                                 float& out0, float& out1, float& h0, float& h1) {
    const uint64_t half2 = f2pack(0.5f, 0.5f), quarter2 = f2pack(0.25f, 0.25f), two2 = f2pack(2.0f, 2.0f);
    const uint64_t st = f2pack(st0, st1), x = f2pack(x0, x1);
    const uint64_t th = f2pack(tanh_fast(hzh0), tanh_fast(hzh1));
    const uint64_t tg = f2pack(tanh_fast(hzg0), tanh_fast(hzg1));
    const uint64_t tp = f2pack(tanh_fast(hzp0), tanh_fast(hzp1));
    const uint64_t sg = f2fma(tg, half2, half2), p = f2fma(tp, half2, half2);
    // g(zh) = 0.5 + max(zh, 0.5 th) = 0.5 + 2 max(zh/2, 0.25 th): every step is exact
    float m0, m1;
    f2unpack(f2mul(th, quarter2), m0, m1);
    const uint64_t gh = f2fma(two2, f2pack(fmaxf(hzh0, m0), fmaxf(hzh1, m1)), half2);
    const uint64_t out = f2fma(sg, f2sub(gh, st), st);
    const uint64_t h = f2fma(p, f2sub(out, x), x);
    f2unpack(out, out0, out1);
    f2unpack(h, h0, h1);
}

struct Smem {
    uint8_t* base;
    int off_s, off_t, off_bias, off_bars, off_misc, b_slot_bytes;
    template <bool PAIR, int GAME, int HID> __device__ __forceinline__ void layout() {
        using C = Cfg<PAIR, GAME, HID>;
        off_s = C::kOffS; off_t = C::kOffT;
        off_bias = C::kOffBias; off_bars = C::kOffBars; off_misc = C::kOffMisc; b_slot_bytes = C::kBSlot;
    }
    __device__ __forceinline__ uint32_t bar(int i) const { return smem_u32(base + off_bars + i * 8); }
    __device__ __forceinline__ uint8_t* b_ring() const { return base; }
    __device__ __forceinline__ uint8_t* s_slot(int s) const { return base + off_s + s * kSSlot; }
    // record slots 0 and 1 have room of their own, slot s >= 2 is state slot s - 2
    __device__ __forceinline__ uint8_t* r_slot(int s) const {
        return s < kOwnRSlots ? base + off_t + s * kRSlot : base + off_s + (s - kOwnRSlots) * kSSlot;
    }
    __device__ __forceinline__ uint8_t* t_buf() const { return base + off_t; }
    __device__ __forceinline__ float* bias() const { return reinterpret_cast<float*>(base + off_bias); }
    __device__ __forceinline__ uint32_t* tmem_base() const { return reinterpret_cast<uint32_t*>(base + off_misc); }
    __device__ __forceinline__ volatile uint32_t* abort_flag() const {
        return reinterpret_cast<volatile uint32_t*>(base + off_misc + 4);
    }
};

// Hooks of a profiling build: a header given with -include may define them to sum clock64
// deltas per phase; in the library they expand to nothing.
#ifndef CFX_MARK
#define CFX_MARK_INIT(role)
#define CFX_MARK(bucket)
#define CFX_MARK_FLUSH()
#endif

// every role runs in its own function: a failed (timed-out) wait returns to the common exit
// Copy threads and worker warps poll with try_wait (suspends while not ready).
// Measured alternatives, all slower on B200: one polling lane per worker warp plus a shuffle
// (+25 % kernel time), a test_wait probe in front of the loop (+6 %).
#define CFX_WAIT(barid, parity, code) \
    if (!mbar_wait(sm.bar(barid), (parity), sm.abort_flag(), (code))) return
#define CFX_WAITW(barid, parity, code) CFX_WAIT(barid, parity, code)
// the three copy-issuing threads (weights, loads, stores): no back-off between probes
#define CFX_WAIT_FAST(barid, parity, code) \
    if (!mbar_wait<false>(sm.bar(barid), (parity), sm.abort_flag(), (code))) return
// The MMA role runs on ONE thread; the other lanes of its warp go straight to the exit.  (A
// converged warp with an elected lane, one shuffle per wait and a __syncwarp per stage, was
// 10 % slower end to end.)  It polls with test_wait: it never suspends.  The first probe is
// inline: almost every wait of this thread finds its barrier complete (5 failed probes in the
// 32 weight waits of a tile), and the bounded loop costs ~150 cycles more than one probe.
#define CFX_WAIT_LEADER(barid, parity, code)                                          \
    if (!mbar_test_wait(sm.bar(barid), (parity)) &&                                   \
        !mbar_wait_spin(sm.bar(barid), (parity), sm.abort_flag(), (code)))            \
    return

// Record ring schedule (full game).  Fill kc of a tile carries record bytes [64 kc, 64 kc + 64)
// of all 128 envs.  Worker warpgroup 1 is free as soon as the previous tile's heads are done,
// warpgroup 0 samples the previous tile's actions first: warpgroup 1 converts chunks 0, 1, 2 and
// then the even chunks, warpgroup 0 the odd chunks from 3 on, so that the MMA thread, which
// consumes the chunks in order, finds the two warpgroups working on neighbouring chunks.  Each
// warpgroup has three ring slots of its own, filled in order by one thread (the load thread for
// warpgroup 1, the store thread for warpgroup 0: see role_loads).  With one producer and one consumer per slot, both sides keep a slot's phase
// as a running count of their own uses.  (The classic game shares its record buffer between
// the warpgroups: even chunks warpgroup 1, odd ones warpgroup 0.)
__device__ __forceinline__ int rec_owner(int kc) { return (kc & 1) ^ 1; }
constexpr int kHeadStart = 3, kWgRSlots = 3;
__device__ __forceinline__ int full_owner(int kc) { return kc < kHeadStart ? 1 : ((kc & 1) ^ 1); }
__device__ __forceinline__ int full_first(int wg) { return wg == 1 ? 0 : kHeadStart; }
// the chunk the same warpgroup converts after chunk kc (beyond the last chunk: none)
__device__ __forceinline__ int full_next(int kc) { return kc < kHeadStart - 1 ? kc + 1 : kc + 2; }
// position of chunk kc in its warpgroup's sequence, and the ring slot it lands in
__device__ __forceinline__ int full_index(int kc) {
    return kc < kHeadStart ? kc : ((kc & 1) ? (kc - kHeadStart) >> 1 : kHeadStart + ((kc - kHeadStart - 1) >> 1));
}
__device__ __forceinline__ int full_rslot(int kc) {
    return (full_owner(kc) == 1 ? 0 : kWgRSlots) + full_index(kc) % kWgRSlots;
}

// Software prefetch into L2.  The rings are far too small to cover HBM latency at the rate the
// encoder and the cell consume, so every byte a ring will load is requested from HBM ahead of
// time in 16 KB pieces, and the ring loads then hit L2 (hundreds of cycles instead of
// thousands).  The load thread issues the pieces, a few with every pair of state boxes it
// loads, which spreads them over the gate phases (one burst per tile delayed that tile's own loads by
// thousands of cycles) and keeps the distance to the use short (a whole tile ahead, part of
// the data had been evicted again):
//   while layer l < L-1 runs   -> the state rows of layer l+1 of the same tile
//   while the last layer runs  -> the records and the layer-0 state rows of the CTA's next tile
constexpr uint32_t kL2Piece = 16384;
__device__ __forceinline__ void l2_prefetch_rows(const uint8_t* base, uint32_t bytes, int piece) {
    const uint32_t o = (uint32_t)piece * kL2Piece;
    if (o < bytes) bulk_prefetch_l2(base + o, min(kL2Piece, bytes - o));
}
template <int HID>
__device__ __forceinline__ void l2_prefetch_for_box(const Params& P, int tile, int l, int j) {
    CFX_DIMS(HID);
    if (tile >= P.num_tiles) return;   // the filler tile of an odd pair
    if (l < P.L - 1) {
        const int rows = min(kTile, P.n - tile * kTile);
        l2_prefetch_rows(reinterpret_cast<const uint8_t*>(
                             P.state + ((size_t)(l + 1) * P.n + (size_t)tile * kTile) * kH),
                         (uint32_t)rows * kH * 4, j);
    } else {
        const int t = tile + gridDim.x;
        if (t >= P.num_tiles) return;
        const int rows = min(kTile, P.n - t * kTile);
        // a tile's records are up to eight pieces: spread over the boxes of the layer
        constexpr int kRecPieces = 8 / kStateItems;
#pragma unroll
        for (int q = 0; q < kRecPieces; q++)
            l2_prefetch_rows(P.records + (size_t)t * kTile * P.rec_bytes, (uint32_t)rows * P.rec_bytes,
                             j * kRecPieces + q);
        l2_prefetch_rows(reinterpret_cast<const uint8_t*>(P.state + (size_t)t * kTile * kH),
                         (uint32_t)rows * kH * 4, j);
    }
}

// ------------------------------------------------------------------ producer roles
// Weight stages: the image is laid out in consumption order, so stage s of a tile starts
// where stage s-1 ended; every tile replays the same sequence (it stays L2 resident).
// In a CTA pair every CTA stages its own half of the rows of each
// stage (contiguous in the image) with a tensor copy whose completion is counted on the even
// CTA's "full" barrier, where the MMA thread waits; one CTA per tile uses plain bulk copies.
template <bool PAIR, int GAME, int HID>
__device__ __forceinline__ void role_weight_loads(const Smem& sm, const Params& P, int lane,
                                                  uint32_t rank, uint32_t bar0_cta0) {
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kEncStages = Gm<GAME>::kEncBlocks / kStageBlocks;
    const int stages_gate = P.L * kSlices * (kKBlocks / kStageBlocks);
    const size_t enc_bytes = fused::enc_bytes<GAME, HID>();
    // One lane walks the launch-wide stage sequence: the slots come free in the order they were
    // filled.  (One lane per slot, diverged inside one warp, delivered stages late: a lane whose
    // slot had come free waited for the warp to leave another lane's suspended wait.)
    const int per_tile = kEncStages + stages_gate + 1;
    int tile = P.tile_begin + blockIdx.x, s = 0;
    int slot = 0;
    uint32_t par = 1;   // parity of the "empty" phase to wait for: the first pass finds every slot free
    (void)lane;
    CFX_MARK_INIT(3);
    for (; tile < P.num_tiles_loop;) {
        uint32_t bytes;
        size_t off;
        if (s < kEncStages) {
            bytes = kEncCopyBytes; off = (size_t)s * kEncCopyBytes;
        } else if (s < kEncStages + stages_gate) {
            bytes = kGateStageBytes; off = enc_bytes + (size_t)(s - kEncStages) * kGateStageBytes;
        } else {
            bytes = head_bytes<GAME, HID>(PAIR);
            off = enc_bytes + (size_t)stages_gate * kGateStageBytes;
        }
        CFX_WAIT_FAST(B_EMPTY + slot, par, W_B_EMPTY);
        CFX_MARK(1);
        const uint32_t dst = smem_u32(sm.b_ring() + slot * C::kBSlot);
        if (PAIR) {
            // Each CTA copies its half of the stage into its own shared memory; both copies are
            // counted on the EVEN CTA's "full" barrier (where the MMA thread waits), which
            // expects the bytes of the whole stage.  The odd CTA needs no barrier of its own
            // and no forwarding hop.
            const int region = s < kEncStages ? 0 : (s < kEncStages + stages_gate ? 1 : 2);
            const size_t base = region == 0 ? 0 : (region == 1 ? enc_bytes : enc_bytes + (size_t)stages_gate * kGateStageBytes);
            const uint32_t half = bytes >> 1;
            const int y = (int)((off - base + (size_t)rank * half) >> 7);   // rows of 128 bytes
            if (rank == 0) mbar_arrive_expect_tx(sm.bar(B_FULL + slot), bytes);
            tensor_g2s_2d_pair(dst, &P.w_map[region], 0, y, bar0_cta0 + 8u * (uint32_t)(B_FULL + slot));
        } else {
            mbar_arrive_expect_tx(sm.bar(B_FULL + slot), bytes);
            bulk_g2s(dst, P.image + off, bytes, sm.bar(B_FULL + slot));
        }
        CFX_MARK(2);
        if (++s == per_tile) { s = 0; tile += gridDim.x; }
        if (++slot == C::kNB) { slot = 0; par ^= 1u; }
    }
    CFX_MARK_FLUSH();
}

// Records: the [n][996] byte array is viewed as [n/4][3984] (four records per 16-byte
// aligned row); env 4g+i of a tile sits in row g at byte 996 i.  A 64-byte chunk of all 128
// records is fetched as four boxes (one per i) of 32 rows x 80 bytes starting at the 16-byte
// boundary below 996 i + 64 c (the last chunk's boxes reach past the row: zero fill).
__device__ __forceinline__ void record_fill(const Smem& sm, const Params& P, int tile, int kc, int slot) {
    mbar_arrive_expect_tx(sm.bar(R_FULL + slot), kRSlot);
    const uint32_t slot_addr = smem_u32(sm.r_slot(slot));
#pragma unroll
    for (int i = 0; i < 4; i++)
        tensor_g2s_2d(slot_addr + i * kRBoxBytes, &P.rec_map, (kRec * i + 64 * kc) & ~15, tile * 32,
                      sm.bar(R_FULL + slot));
}

// State boxes: layer l, tile rows, 32 units -> one 16 KB box, 128-byte swizzled; box j of a
// layer belongs to slice j / 2 and worker warpgroup j & 1, and box b of a tile uses ring slot
// b % 4.  The workers replace a box's contents with the new state in place; it is then written
// back (rows beyond n are clipped by the tensor map) and the slot is loaded again.
//
// Two threads in two warps feed the rings, each a plain sequence of waits and copies.  (Several
// lanes of one warp, one per ring slot, each in its own loop, ran at a fraction of that speed:
// a lane whose barrier had completed took 600-700 cycles to get from one statement to the
// next while the warp served the other lanes.)
//   load thread:  per tile, the record fills of worker warpgroup 1, then the state box loads;
//   store thread: per tile, the record fills of worker warpgroup 0, then the state box stores.
// The record phase and the state phase of a tile do not overlap in time, so neither thread
// holds the other's work up.  The load thread takes a state slot when the store thread reports
// that the previous box has been read out of it (S_FREE); that includes state slot 0 before it
// is used as warpgroup 1's third record slot.  The store thread's own record slots are state
// slots 1-3, free once its stores of the previous tile have been read.
template <bool PAIR, int GAME, int HID>
__device__ __forceinline__ void role_loads(const Smem& sm, const Params& P) {
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kNS = C::kNS;
    static_assert(kStateItems % kNS == 0 && (GAME != CFX_GAME_FULL || C::kOwn == kWgRSlots - 1),
                  "box b of a tile uses slot b % kNS; warpgroup 1's third record slot is state slot 0");
    uint32_t it = 0;
    uint32_t epar = (1u << kNRMax) - 1u;   // record slots: parity of the "empty" phase to wait for
    uint32_t fpar = (1u << kNS) - 1u;      // state slots: parity of the "free" phase to wait for
    CFX_MARK_INIT(4);
    for (int tile = P.tile_begin + blockIdx.x; tile < P.num_tiles_loop; tile += gridDim.x, it++) {
        if constexpr (GAME == CFX_GAME_CLASSIC) {
            // classic: the records of the whole tile are one box, 32 rows of four 148-byte
            // records (a [n/4][148] array of 32-bit words)
            CFX_WAIT_FAST(T_EMPTY, (it & 1) ^ 1, W_T_EMPTY);
            mbar_arrive_expect_tx(sm.bar(T_FULL), 128 * kClassicRec);
            tensor_g2s_2d(smem_u32(sm.t_buf()), &P.rec_map, 0, tile * 32, sm.bar(T_FULL));
        } else {
            for (int kc = full_first(1); kc < Gm<GAME>::kEncChunks; kc = full_next(kc)) {
                const int slot = full_rslot(kc);
                if (slot >= C::kOwn && full_index(kc) < kWgRSlots) {   // first fill of the tile into state slot 0
                    CFX_WAIT_FAST(S_FREE + slot - C::kOwn, (fpar >> (slot - C::kOwn)) & 1u, W_S_FREE);
                    fpar ^= 1u << (slot - C::kOwn);
                }
                CFX_WAIT_FAST(R_EMPTY + slot, (epar >> slot) & 1u, W_R_EMPTY);
                epar ^= 1u << slot;
                record_fill(sm, P, tile, kc, slot);
            }
        }
        int b = 0;
        for (int l = 0; l < P.L; l++) {
            for (int j = 0; j < kStateItems; j++, b++) {
                const int slot = b % kNS;
                // the first box of the tile: every record of the tile has been expanded
                if (C::kAlias && b == 0) CFX_WAIT_FAST(REC_DONE, it & 1, W_REC_DONE);
                if (!(C::kAlias && b == 0)) {   // (slot 0 was taken for the records already)
                    CFX_WAIT_FAST(S_FREE + slot, (fpar >> slot) & 1u, W_S_FREE);
                    fpar ^= 1u << slot;
                }
                CFX_MARK(1);
                mbar_arrive_expect_tx(sm.bar(S_FULL + slot), kSSlot);
                tensor_g2s_2d(smem_u32(sm.s_slot(slot)), &P.state_map[l], j * kHalfUnits, tile * kTile,
                              sm.bar(S_FULL + slot));
                CFX_MARK(2);
                // the L2 prefetches that go with the two boxes of a slice, after both loads
                if (j & 1) {
                    l2_prefetch_for_box<HID>(P, tile, l, j - 1);
                    l2_prefetch_for_box<HID>(P, tile, l, j);
                }
            }
        }
    }
    CFX_MARK_FLUSH();
}

template <bool PAIR, int GAME, int HID>
__device__ __forceinline__ void role_stores(const Smem& sm, const Params& P) {
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kNS = C::kNS;
    static_assert(kStateItems % 2 == 0, "the two boxes of a slice are written back together");
    uint32_t epar = (1u << kNRMax) - 1u;   // record slots: parity of the "empty" phase to wait for
    uint32_t spar = 0;                     // state slots: parity of the "new state ready" phase
    CFX_MARK_INIT(5);
    for (int tile = P.tile_begin + blockIdx.x; tile < P.num_tiles_loop; tile += gridDim.x) {
        if constexpr (GAME == CFX_GAME_FULL) {
            for (int kc = full_first(0); kc < Gm<GAME>::kEncChunks; kc = full_next(kc)) {
                const int slot = full_rslot(kc);
                CFX_WAIT_FAST(R_EMPTY + slot, (epar >> slot) & 1u, W_R_EMPTY);
                epar ^= 1u << slot;
                record_fill(sm, P, tile, kc, slot);
            }
        }
        int b = 0;
        for (int l = 0; l < P.L; l++) {
            for (int j = 0; j < kStateItems; j++, b++) {
                const int slot = b % kNS;
                CFX_WAIT_FAST(ST_READY + slot, (spar >> slot) & 1u, W_ST_READY);
                spar ^= 1u << slot;
                CFX_MARK(3);
                tensor_s2g_2d(&P.state_map[l], smem_u32(sm.s_slot(slot)), j * kHalfUnits, tile * kTile);
                bulk_commit_group();
                if (j & 1) {
                    // a slot is free as soon as its box has been read out of shared memory
                    bulk_wait_group_read<1>();
                    mbar_arrive(sm.bar(S_FREE + (b - 1) % kNS));
                    bulk_wait_group_read<0>();
                    mbar_arrive(sm.bar(S_FREE + slot));
                    CFX_MARK(4);
                }
            }
        }
    }
    bulk_wait_group<0>();
    CFX_MARK_FLUSH();
}

// ------------------------------------------------------------------ MMA role
// One thread issues every MMA of the CTA.  The tensor pipe queues about eight MMAs, so the
// issuer runs ahead of it as long as its own loop is short: descriptors are one add away from
// a per-slot base and every K-step loop is fully unrolled (rebuilding descriptors per MMA
// measured ~150 cycles per instruction on B200, against 45-50 for the bare instruction), and
// MMAs are as wide as the tensor memory budget allows (N = 192 / 256).
#define MMA_TS(...)                                  \
    do {                                             \
        if (PAIR) mma_f16_ts_pair(__VA_ARGS__);      \
        else mma_f16_ts(__VA_ARGS__);                \
    } while (0)
// commits: in a pair they arrive on the barrier of BOTH CTAs
#define MMA_COMMIT(bar)                  \
    do {                                 \
        if (PAIR) mma_commit_pair(bar);  \
        else mma_commit(bar);            \
    } while (0)
template <typename T16, bool PAIR, int GAME, int HID>
__device__ __forceinline__ void role_mma(const Smem& sm, const Params& P, uint32_t tmem) {
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kEncChunks = Gm<GAME>::kEncChunks;
    constexpr int kNB = C::kNB, kBSlot = C::kBSlot;
    constexpr uint32_t fmt = Op16<T16>::kFmt;
    constexpr uint32_t idesc_enc = make_idesc(fmt, C::kM, kH);
    constexpr uint32_t idesc_gate = make_idesc(fmt, C::kM, 3 * kSliceUnits);
    constexpr uint32_t idesc_head = make_idesc(fmt, C::kM, C::kHeadRows);
    // descriptor steps (16-byte units) between the two blocks of a stage: a CTA of a pair
    // holds half of each block's rows
    constexpr uint32_t kEncBlkStep = ((PAIR ? kH / 2 : kH) * 128) >> 4;
    constexpr uint32_t kGateBlkStep = ((PAIR ? 3 * kSliceUnits / 2 : 3 * kSliceUnits) * 128) >> 4;
    const uint64_t bdesc0 = smem_desc_sw128(smem_u32(sm.b_ring()));
    uint32_t acnt = 0, akb_use = 0, gcnt = 0, tcnt = 0;
    // position in the weight ring of the stage being consumed: slot and phase parity, advanced
    // incrementally (a division per stage on this thread would sit on the critical path)
    int bslot = 0;
    uint32_t bpar = 0;
    auto b_advance = [&]() {
        if (++bslot == kNB) { bslot = 0; bpar ^= 1u; }
    };
    // The "full" barriers of the NEXT stage are probed before the current stage's MMAs are
    // issued, so that the probe's shared-memory round trip (~150 cycles on this thread) runs
    // under the MMA issue; only a failed probe falls into the bounded wait.  Probing one stage
    // early is sound: the previous use of that slot has already been consumed by this thread,
    // so its barrier is at most one phase behind.
    // The probes are deferred ones (CFX_PROBE): their result is read a stage later.
    auto probe_b_next = [&]() {
        const bool wrap = bslot + 1 == kNB;
        CFX_PROBE(cfx_p_b, sm.bar(B_FULL + (wrap ? 0 : bslot + 1)), wrap ? bpar ^ 1u : bpar);
    };
    auto probe_a = [&](uint32_t cnt) {
        CFX_PROBE(cfx_p_a, sm.bar(AEXP_FULL + (int)(cnt % kAexpSlots)), (cnt / kAexpSlots) & 1);
    };
#define CFX_WAIT_PROBED(name, barid, parity, code)                                                  \
    {                                                                                               \
        uint32_t ready_;                                                                            \
        CFX_PROBE_READ(name, ready_);                                                               \
        if (ready_ == 0 && !mbar_wait_spin(sm.bar(barid), (parity), sm.abort_flag(), (code))) return; \
    }
    CFX_MARK_INIT(0);
    for (int tile = P.tile_begin + blockIdx.x; tile < P.num_tiles_loop; tile += gridDim.x, tcnt++) {
        CFX_MARK(0);
        // the encoder accumulator overlaps the head accumulator of the previous tile:
        // wait until the sampler threads have read it
        CFX_WAIT_LEADER(H_EMPTY, (tcnt & 1) ^ 1, W_H_EMPTY);
        probe_a(acnt);
        CFX_PROBE(cfx_p_b, sm.bar(B_FULL + bslot), bpar);
        // ---- encoder: N = kH units; one weight stage (two blocks of 64 K columns) per two
        // chunks, except the full game's last stage, which four short chunks consume
        // one operand chunk: wait for it, issue its K steps against the block at descriptor bd
#define CFX_ENC_CHUNK(kc, bd, ksteps)                                                              \
        {                                                                                          \
            const int as = acnt % kAexpSlots;                                                      \
            CFX_WAIT_PROBED(cfx_p_a, AEXP_FULL + as, (acnt / kAexpSlots) & 1, W_AEXP_FULL);        \
            CFX_MARK(2);                                                                           \
            tc_fence_after_sync();                                                                 \
            if ((kc) + 1 < kEncChunks) probe_a(acnt + 1);                                          \
            const uint32_t a_col = tmem + kColAexp + as * 32;                                      \
            if ((kc) == 0) MMA_TS(tmem + kColAcc, a_col, (bd), idesc_enc, 0);                      \
            else MMA_TS(tmem + kColAcc, a_col, (bd), idesc_enc, 1);                                \
            if ((ksteps) > 1) {                                                                    \
                MMA_TS(tmem + kColAcc, a_col + 8, (bd) + 2, idesc_enc, 1);                         \
                MMA_TS(tmem + kColAcc, a_col + 16, (bd) + 4, idesc_enc, 1);                        \
            }                                                                                      \
            if ((ksteps) > 3) MMA_TS(tmem + kColAcc, a_col + 24, (bd) + 6, idesc_enc, 1);          \
            MMA_COMMIT(sm.bar(AEXP_EMPTY + as));                                                   \
            acnt++;                                                                                \
            CFX_MARK(4);                                                                           \
        }
        constexpr int kFullStages = GAME == CFX_GAME_FULL ? 6 : kEncChunks / kStageBlocks;
        for (int kp = 0; kp < kFullStages; kp++) {
            const int slot = bslot;
            CFX_WAIT_PROBED(cfx_p_b, B_FULL + slot, bpar, W_B_FULL);
            CFX_MARK(3);
            probe_b_next();
            b_advance();
            const uint64_t bd0 = bdesc0 + (uint64_t)(slot * (kBSlot >> 4));
#pragma unroll
            for (int c2 = 0; c2 < kStageBlocks; c2++) {
                const int kc = kStageBlocks * kp + c2;
                // the classic game's last chunk carries one feature (one K step)
                const int ksteps = GAME == CFX_GAME_CLASSIC && kc == kEncChunks - 1 ? 1 : 4;
                CFX_ENC_CHUNK(kc, bd0 + (uint64_t)(c2 * kEncBlkStep), ksteps);
            }
            MMA_COMMIT(sm.bar(B_EMPTY + slot));
        }
        if constexpr (GAME == CFX_GAME_FULL) {
            // blocks 12 and 13: chunk 12 = K columns 0-47 of block 12 (three K steps), chunk 13
            // = columns 48-63; chunk 14 = columns 0-15 of block 13, chunk 15 = columns 16-31
            const int slot = bslot;
            CFX_WAIT_PROBED(cfx_p_b, B_FULL + slot, bpar, W_B_FULL);
            CFX_MARK(3);
            probe_b_next();
            b_advance();
            const uint64_t bd0 = bdesc0 + (uint64_t)(slot * (kBSlot >> 4));
            CFX_ENC_CHUNK(12, bd0, 3);
            CFX_ENC_CHUNK(13, bd0 + 6, 1);
            CFX_ENC_CHUNK(14, bd0 + (uint64_t)kEncBlkStep, 1);
            CFX_ENC_CHUNK(15, bd0 + (uint64_t)(kEncBlkStep + 2), 1);
            MMA_COMMIT(sm.bar(B_EMPTY + slot));
        }
#undef CFX_ENC_CHUNK
        MMA_COMMIT(sm.bar(ACC_FULL));

        // ---- MinGRU layers: 4 slices of 64 units, one stage per two K blocks, N = 192 (zh|zg|zp)
        for (int l = 0; l < P.L; l++, akb_use++) {
            const uint32_t a_cur = tmem + ((l & 1) ? kColA1 : kColA0);
            for (int j = 0; j < kSlices; j++, gcnt++) {
                CFX_WAIT_LEADER(G_EMPTY, (gcnt & 1) ^ 1, W_G_EMPTY);
                CFX_MARK(5);
                // The gate accumulator overlaps the encoder accumulator: the first gate MMA of a
                // tile waits until every worker warp has moved its part of it to registers.
                // (An early version waited only for the K block it multiplied while a warpgroup
                // was still reading the accumulator: about one launch in a hundred changed 32
                // rows of one tile.)
                if (l == 0 && j == 0) {
                    CFX_WAIT_LEADER(ACC_READ, tcnt & 1, W_ACC_READ);
                    CFX_MARK(9);
                }
#pragma unroll
                for (int kp = 0; kp < kKBlocks / kStageBlocks; kp++) {
                    const int slot = bslot;
                    CFX_WAIT_PROBED(cfx_p_b, B_FULL + slot, bpar, W_B_FULL);
                    CFX_MARK(6);
                    probe_b_next();
                    b_advance();
                    const uint64_t bd0 = bdesc0 + (uint64_t)(slot * (kBSlot >> 4));
#pragma unroll
                    for (int c2 = 0; c2 < kStageBlocks; c2++) {
                        const int kb = kStageBlocks * kp + c2;
                        // the layer's input arrives K block by K block (slice kb of the previous layer)
                        if (j == 0) {
                            CFX_WAIT_LEADER(A_KB + kb, akb_use & 1, W_A_KB);
                            CFX_MARK(9);
                        }
                        tc_fence_after_sync();
#pragma unroll
                        for (int ks = 0; ks < 4; ks++)
                            MMA_TS(tmem + kColG, a_cur + kb * 32 + ks * 8,
                                   bd0 + (uint64_t)(c2 * kGateBlkStep + 2 * ks), idesc_gate,
                                   (kb | ks) != 0 ? 1u : 0u);
                    }
                    MMA_COMMIT(sm.bar(B_EMPTY + slot));
                    CFX_MARK(7);
                }
                MMA_COMMIT(sm.bar(G_FULL));
            }
        }
        // ---- heads: N = 48 (64 in a pair), one stage with all K blocks
        {
            const uint32_t a_cur = tmem + ((P.L & 1) ? kColA1 : kColA0);
            const int slot = bslot;
            CFX_WAIT_PROBED(cfx_p_b, B_FULL + slot, bpar, W_B_FULL);
            b_advance();
            const uint64_t bd = bdesc0 + (uint64_t)(slot * (kBSlot >> 4));
            // K block kb of the last layer's output is complete when slice kb's cells are done
#pragma unroll
            for (int kb = 0; kb < kKBlocks; kb++) {
                CFX_WAIT_LEADER(A_KB + kb, akb_use & 1, W_A_KB);
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    MMA_TS(tmem + kColHead, a_cur + kb * 32 + ks * 8,
                           bd + (uint64_t)((kb * C::kHeadKbBytes + ks * 32) >> 4), idesc_head,
                           (kb | ks) != 0 ? 1u : 0u);
            }
            akb_use++;
            MMA_COMMIT(sm.bar(B_EMPTY + slot));
            MMA_COMMIT(sm.bar(H_FULL));
            CFX_MARK(8);
        }
    }
    CFX_MARK_FLUSH();
}

// ------------------------------------------------------------------ worker role
// Eight warps, two per TMEM lane quarter (wg 0 / wg 1); thread (quarter, lane) owns env row
// quarter*32 + lane of the tile in every phase.
template <typename T16, bool PAIR, int GAME, int HID>
__device__ __forceinline__ void role_worker(const Smem& sm, const Params& P, uint32_t tmem,
                                            int warp, int lane, uint32_t bar0_cta0) {
    using Op = Op16<T16>;
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kA = Gm<GAME>::kA, kEncChunks = Gm<GAME>::kEncChunks;
    constexpr int kHeadCols = (kA + 1 + 15) / 16 * 16;   // head accumulator columns that are read
    // barriers the MMA thread waits on live in the even CTA of a pair
    auto arrive_mma = [&](int barid) {
        if (PAIR) mbar_arrive_cluster(bar0_cta0 + 8u * (uint32_t)barid);
        else mbar_arrive(sm.bar(barid));
    };
    const int wg = (warp - kWorkerWarp0) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int gi = row >> 2, ii = row & 3;
    const float* bias = sm.bias();
    const uint32_t rec_row_off = ii * kRBoxBytes + gi * 80;
    uint32_t tcnt = 0, gcnt = 0, it = 0;
    uint32_t rpar = 0;   // full game: phase parity of every record slot, one bit per slot
    // the sampler offset is constant for the launch (the bump happens after every block is done)
    const unsigned long long step0 = P.uniforms == nullptr ? *P.step_ctr : 0ull;
    CFX_MARK_INIT(1 + wg);
    for (int tile = P.tile_begin + blockIdx.x; tile < P.num_tiles_loop; tile += gridDim.x, it++, tcnt++) {
        CFX_MARK(0);
        const int env = tile * kTile + row;
        const bool valid = env < P.n;
        const bool zero_state =
            valid && P.prev_terminals != nullptr && P.prev_terminals[env] != 0.0f;

        // ---- expand: record bytes -> 16-bit operand rows in the TMEM chunk ring.
        // Full game: wg 1 converts chunks 0-2 and the even ones after them, wg 0 (which samples
        // the previous tile's actions first) the odd ones from 3 on.  Classic game: wg 1 converts
        // the even chunks, wg 0 the odd ones.  A warp writes all 32 columns of its rows.
        // Full game: the two barriers of a chunk are probed one chunk ahead, so that the
        // probes' shared-memory round trips (~200 cycles each, also when the barrier is already
        // complete) run under the previous chunk's conversion; only a failed probe falls into
        // the wait loop.  Probing ahead is sound: this warp has itself passed the previous phase
        // of both barriers.
        if (GAME == CFX_GAME_FULL) {
            const int kc0 = full_first(wg);
            const uint32_t acnt0 = it * kEncChunks + kc0;
            CFX_PROBE(cfx_p_ae, sm.bar(AEXP_EMPTY + (int)(acnt0 % kAexpSlots)), ((acnt0 / kAexpSlots) & 1) ^ 1);
            CFX_PROBE(cfx_p_r, sm.bar(R_FULL + full_rslot(kc0)), (rpar >> full_rslot(kc0)) & 1u);
        }
        for (int kc = 0; kc < kEncChunks; kc++) {
            if ((GAME == CFX_GAME_CLASSIC ? rec_owner(kc) : full_owner(kc)) != wg) continue;
            const uint32_t acnt = it * kEncChunks + kc;
            const int as = acnt % kAexpSlots;
            uint32_t ae_ok = 0;
            if (GAME == CFX_GAME_FULL) CFX_PROBE_READ(cfx_p_ae, ae_ok);
            if (ae_ok == 0) CFX_WAITW(AEXP_EMPTY + as, ((acnt / kAexpSlots) & 1) ^ 1, W_AEXP_EMPTY);
            CFX_MARK(2);
            tc_fence_after_sync();
            uint32_t regs[32];
            if constexpr (GAME == CFX_GAME_CLASSIC) {
                // The tile's records are one buffer.  The 1323 one-hot features of a record are
                // a bit stream, 21 bits per view cell (17 block ids + 4 mob bits); a chunk is a
                // 64-bit window of it, built from at most four cells, and every bit becomes
                // 1.0 or 0.0 in the operand type.  Chunk 20 ends with the 21 scalar features
                // (feature order of expand_obs_kernel, craftax_classic.cu:1265-1301), chunk 21
                // holds the sleeping flag alone.
                if (kc <= 1) CFX_WAITW(T_FULL, it & 1, W_T_FULL);   // first chunk of either warpgroup
                const uint8_t* rp = sm.t_buf() + gi * (4 * kClassicRec) + ii * kClassicRec;
                auto cell_bits = [&](int cell) -> uint64_t {
                    if (cell >= kClassicCells) return 0ull;
                    const uint32_t blk = rp[cell], mob = rp[kClassicCells + cell];
                    return (uint64_t)((blk < (uint32_t)kClassicBlocks ? (1u << blk) : 0u) | ((mob & 15u) << kClassicBlocks));
                };
                const int cell0 = (64 * kc) / 21, off0 = 64 * kc - 21 * cell0;
                uint64_t w = 0;
                if (kc < kEncChunks - 1)
                    w = (cell_bits(cell0) >> off0) | (cell_bits(cell0 + 1) << (21 - off0)) |
                        (cell_bits(cell0 + 2) << (42 - off0)) | (cell_bits(cell0 + 3) << (63 - off0));
                const uint32_t wlo = (uint32_t)w, whi = (uint32_t)(w >> 32);
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    regs[q] = ((wlo >> (2 * q)) & 1u) * Op::kOne | ((wlo >> (2 * q + 1)) & 1u) * (Op::kOne << 16);
                    regs[16 + q] = ((whi >> (2 * q)) & 1u) * Op::kOne | ((whi >> (2 * q + 1)) & 1u) * (Op::kOne << 16);
                }
                if (kc == kEncChunks - 2) {   // features 1280..1343: 43 one-hot bits, then 21 scalars
                    float sc[22];
#pragma unroll
                    for (int j2 = 0; j2 < 16; j2++) sc[j2] = (float)(int8_t)rp[2 * kClassicCells + j2] / 10.0f;
                    const int dir = (int8_t)rp[2 * kClassicCells + 16];
#pragma unroll
                    for (int d = 0; d < 4; d++) sc[16 + d] = dir == d + 1 ? 1.0f : 0.0f;
                    sc[20] = *reinterpret_cast<const float*>(rp + 2 * kClassicCells + 18);
                    sc[21] = 0.0f;
                    regs[21] = (regs[21] & 0xFFFFu) | (Op::pack(0.0f, sc[0]) & 0xFFFF0000u);
#pragma unroll
                    for (int q = 22; q < 32; q++) regs[q] = Op::pack(sc[2 * (q - 22) + 1], sc[2 * (q - 22) + 2]);
                } else if (kc == kEncChunks - 1) {   // feature 1344: sleeping
                    regs[0] = rp[2 * kClassicCells + 17] != 0 ? Op::kOne : 0u;
                }
                __syncwarp();
                if (kc >= kEncChunks - 2 && lane == 0) mbar_arrive(sm.bar(T_EMPTY));   // last chunk of this warp
            } else {
                const int slot = full_rslot(kc);
                uint32_t r_ok;
                CFX_PROBE_READ(cfx_p_r, r_ok);
                if (r_ok == 0) CFX_WAITW(R_FULL + slot, (rpar >> slot) & 1u, W_R_FULL);
                rpar ^= 1u << slot;
                CFX_MARK(3);
                if (full_next(kc) < kEncChunks) {
                    const int slot1 = full_rslot(full_next(kc));
                    const uint32_t acnt1 = it * kEncChunks + full_next(kc);
                    CFX_PROBE(cfx_p_ae, sm.bar(AEXP_EMPTY + (int)(acnt1 % kAexpSlots)),
                              ((acnt1 / kAexpSlots) & 1) ^ 1);
                    CFX_PROBE(cfx_p_r, sm.bar(R_FULL + slot1), (rpar >> slot1) & 1u);
                }
                // this env's 64 record bytes of the chunk (4-byte aligned in the slot)
                const uint8_t* src = sm.r_slot(slot) + rec_row_off + ((kRec * ii) & 15);
                auto word = [&](int q) { return *reinterpret_cast<const uint32_t*>(src + 4 * q); };
                if (kc < 12) {          // 64 map bytes
#pragma unroll
                    for (int q = 0; q < 16; q++) Op::bytes4(word(q), regs[2 * q], regs[2 * q + 1]);
                } else {
#pragma unroll
                    for (int q = 0; q < 32; q++) regs[q] = 0u;
                    if (kc == 12) {     // 24 map bytes, then raw floats 0-9
#pragma unroll
                        for (int q = 0; q < 6; q++) Op::bytes4(word(q), regs[2 * q], regs[2 * q + 1]);
#pragma unroll
                        for (int q = 0; q < 5; q++)
                            regs[12 + q] = Op::pack(__uint_as_float(word(6 + 2 * q)), __uint_as_float(word(7 + 2 * q)));
                    } else if (kc < 15) {   // 16 raw floats
#pragma unroll
                        for (int q = 0; q < 8; q++)
                            regs[q] = Op::pack(__uint_as_float(word(2 * q)), __uint_as_float(word(2 * q + 1)));
                    } else {            // the last 9 raw floats; the record ends after them
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            regs[q] = Op::pack(__uint_as_float(word(2 * q)), __uint_as_float(word(2 * q + 1)));
                        regs[4] = Op::pack(__uint_as_float(word(8)), 0.0f);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sm.bar(R_EMPTY + slot));
                    // this warp has read its last record byte of the tile; when all have, the
                    // state boxes may come in
                    if (full_next(kc) >= kEncChunks) mbar_arrive(sm.bar(REC_DONE));
                }
            }
            {
                uint32_t lo[16], hi[16];
#pragma unroll
                for (int q = 0; q < 16; q++) { lo[q] = regs[q]; hi[q] = regs[16 + q]; }
                tmem_st16(tmem + lane_base + kColAexp + as * 32, lo);
                tmem_st16(tmem + lane_base + kColAexp + as * 32 + 16, hi);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) arrive_mma(AEXP_FULL + as);
            CFX_MARK(4);
        }

        // ---- encoder epilogue: accumulator + bias -> layer-0 input A0.  Like in the gate
        // layers, warpgroup wg handles units [64 kb + 32 wg, 64 kb + 32 wg + 32) of K block kb.
        // The whole accumulator goes to registers first and is handed back at once (ACC_READ):
        // the gate accumulator overlaps it, and the first slice's MMAs then start on K block 0
        // while the later blocks are still being converted.
        CFX_WAITW(ACC_FULL, tcnt & 1, W_ACC_FULL);
        CFX_MARK(5);
        tc_fence_after_sync();
        {
            uint32_t acc[kKBlocks][32];
#pragma unroll
            for (int kb = 0; kb < kKBlocks; kb++) {
                uint32_t t0[16], t1[16];
                tmem_ld16(tmem + lane_base + kColAcc + kSliceUnits * kb + kHalfUnits * wg, t0);
                tmem_ld16(tmem + lane_base + kColAcc + kSliceUnits * kb + kHalfUnits * wg + 16, t1);
#pragma unroll
                for (int q = 0; q < 16; q++) { acc[kb][q] = t0[q]; acc[kb][16 + q] = t1[q]; }
            }
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) arrive_mma(ACC_READ);
#pragma unroll
            for (int kb = 0; kb < kKBlocks; kb++) {
                uint32_t pk[16];
                const float* bb = bias + kSliceUnits * kb + kHalfUnits * wg;
#pragma unroll
                for (int q = 0; q < 16; q++)
                    pk[q] = Op::pack(__uint_as_float(acc[kb][2 * q]) + bb[2 * q],
                                     __uint_as_float(acc[kb][2 * q + 1]) + bb[2 * q + 1]);
                tmem_st16(tmem + lane_base + kColA0 + (kSliceUnits / 2) * kb + (kHalfUnits / 2) * wg, pk);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) arrive_mma(A_KB + kb);
            }
        }
        CFX_MARK(1);

        // ---- MinGRU layers: both warpgroups work on every 64-unit slice; wg handles units
        // [64 j + 32 wg, 64 j + 32 wg + 32) = state box 2 j + wg of the layer
        // Here too the next barrier is probed while other work runs: the state box while the
        // accumulator is read, the next accumulator (or the heads) while the cell's last stores
        // drain.
        CFX_PROBE_CLEAR(cfx_p_g);
        for (int l = 0; l < P.L; l++) {
            const uint32_t a_cur = tmem + lane_base + ((l & 1) ? kColA1 : kColA0);
            const uint32_t a_next = tmem + lane_base + ((l & 1) ? kColA0 : kColA1);
            for (int j = 0; j < kSlices; j++, gcnt++) {
                {
                    uint32_t g_ok;
                    CFX_PROBE_READ(cfx_p_g, g_ok);
                    if (g_ok == 0) CFX_WAITW(G_FULL, gcnt & 1, W_G_FULL);
                }
                CFX_MARK(6);
                tc_fence_after_sync();
                const int box = 2 * j + wg;
                const uint32_t scnt = (it * P.L + l) * kStateItems + box;
                constexpr int kNS = C::kNS;
                const int slot = scnt % kNS;
                CFX_PROBE(cfx_p_s, sm.bar(S_FULL + slot), (scnt / kNS) & 1);
                const uint32_t gcol = tmem + lane_base + kColG + kHalfUnits * wg;
                uint8_t* rbase = sm.s_slot(slot) + (row >> 3) * 1024 + (row & 7) * 128;
                const int xr = row & 7;
                // this thread's 96 gate columns and 32 layer inputs go to registers at once, so
                // the accumulator is handed back to the MMA warp right away
                uint32_t zh[32], zg[32], zp[32], xin[16];
                {
                    uint32_t t0[16], t1[16];
                    tmem_ld16(gcol, t0);
                    tmem_ld16(gcol + 16, t1);
#pragma unroll
                    for (int q = 0; q < 16; q++) { zh[q] = t0[q]; zh[16 + q] = t1[q]; }
                    tmem_ld16(gcol + kSliceUnits, t0);
                    tmem_ld16(gcol + kSliceUnits + 16, t1);
#pragma unroll
                    for (int q = 0; q < 16; q++) { zg[q] = t0[q]; zg[16 + q] = t1[q]; }
                    tmem_ld16(gcol + 2 * kSliceUnits, t0);
                    tmem_ld16(gcol + 2 * kSliceUnits + 16, t1);
#pragma unroll
                    for (int q = 0; q < 16; q++) { zp[q] = t0[q]; zp[16 + q] = t1[q]; }
                    tmem_ld16(a_cur + 16 * box, xin);
                    tmem_wait_ld();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) arrive_mma(G_EMPTY);
                CFX_MARK(7);
                {
                    uint32_t s_ok;
                    CFX_PROBE_READ(cfx_p_s, s_ok);
                    if (s_ok == 0) CFX_WAITW(S_FULL + slot, (scnt / kNS) & 1, W_S_FULL);
                }
                CFX_MARK(8);
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    uint32_t hn[8];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int u = 16 * hf + 4 * q;  // first of four units
                        float4* sp = reinterpret_cast<float4*>(rbase + (((4 * hf + q) ^ xr) << 4));
                        float4 st = *sp;
                        if (zero_state) st = make_float4(0.f, 0.f, 0.f, 0.f);
                        // optional BPTT record of the post-zero input state (what the reference's
                        // k_mingru_epi_fwd stores, craftax_full.cu:9370-9375): [L][n][256] fp32
                        if (P.r_state != nullptr && valid) {
                            const size_t o = ((size_t)l * P.n + env) * kH + kSliceUnits * j + kHalfUnits * wg + u;
                            if (P.r_state_bf16) {
                                __nv_bfloat162 lo2 = __floats2bfloat162_rn(st.x, st.y);
                                __nv_bfloat162 hi2 = __floats2bfloat162_rn(st.z, st.w);
                                uint2 v2;
                                v2.x = *reinterpret_cast<uint32_t*>(&lo2);
                                v2.y = *reinterpret_cast<uint32_t*>(&hi2);
                                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(P.r_state) + o) = v2;
                            } else {
                                *reinterpret_cast<float4*>(P.r_state + o) = st;
                            }
                        }
                        const float2 x01 = Op::unpack(xin[u / 2]), x23 = Op::unpack(xin[u / 2 + 1]);
                        float4 out;
                        float h0, h1, h2, h3;
                        mingru_cell_pair(__uint_as_float(zh[u]), __uint_as_float(zh[u + 1]),
                                         __uint_as_float(zg[u]), __uint_as_float(zg[u + 1]),
                                         __uint_as_float(zp[u]), __uint_as_float(zp[u + 1]),
                                         st.x, st.y, x01.x, x01.y, out.x, out.y, h0, h1);
                        mingru_cell_pair(__uint_as_float(zh[u + 2]), __uint_as_float(zh[u + 3]),
                                         __uint_as_float(zg[u + 2]), __uint_as_float(zg[u + 3]),
                                         __uint_as_float(zp[u + 2]), __uint_as_float(zp[u + 3]),
                                         st.z, st.w, x23.x, x23.y, out.z, out.w, h2, h3);
                        *sp = out;
                        hn[2 * q] = Op::pack(h0, h1);
                        hn[2 * q + 1] = Op::pack(h2, h3);
                    }
                    tmem_st8(a_next + 16 * box + 8 * hf, hn);
                }
                // the next accumulator: the heads after the last slice of the last layer
                if (l == P.L - 1 && j == kSlices - 1) CFX_PROBE(cfx_p_g, sm.bar(H_FULL), tcnt & 1);
                else CFX_PROBE(cfx_p_g, sm.bar(G_FULL), (gcnt + 1) & 1);
                tmem_wait_st();
                tc_fence_before_sync();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    arrive_mma(A_KB + j);
                    mbar_arrive(sm.bar(ST_READY + slot));
                }
                CFX_MARK(9);
            }
        }

        // ---- heads + sampler (wg 0: one thread per env; wg 1 only passes the barrier so
        // that its next-tile operand writes cannot overtake the last MMA)
        // the uniform of this env is drawn while the head MMAs run
        float u = 0.0f;
        if (wg == 0 && valid)
            u = P.uniforms != nullptr ? P.uniforms[env]
                                      : philox_uniform(P.seed, P.env_offset + (uint64_t)env, step0);
        {
            uint32_t h_ok;
            CFX_PROBE_READ(cfx_p_g, h_ok);
            if (h_ok == 0) CFX_WAITW(H_FULL, tcnt & 1, W_H_FULL);
        }
        CFX_MARK(10);
        tc_fence_after_sync();
        if (wg == 0) {
            uint32_t hv[kHeadCols];
#pragma unroll
            for (int b = 0; b < kHeadCols / 16; b++) {
                uint32_t t[16];
                tmem_ld16(tmem + lane_base + kColHead + 16 * b, t);
#pragma unroll
                for (int q = 0; q < 16; q++) hv[16 * b + q] = t[q];
            }
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) arrive_mma(H_EMPTY);
            if (valid) {
                float logits[kA];
#pragma unroll
                for (int a = 0; a < kA; a++) logits[a] = __uint_as_float(hv[a]) + bias[kH + a];
                const float value = __uint_as_float(hv[kA]) + bias[kH + kA];
                if constexpr ((kA + 1) % 8 != 4) {
                    float* dst = P.logits_av + (size_t)env * (kA + 1);   // rows are not 16-byte aligned
                    if (P.logits_av != nullptr) {
#pragma unroll
                        for (int a = 0; a < kA; a++) dst[a] = logits[a];
                        dst[kA] = value;
                    }
                } else if (P.logits_av != nullptr) {
                    // A row is 176 bytes: 32-byte aligned for every other env, 16 bytes off for the
                    // ones between.  It goes out as five 32-byte stores and one 16-byte store (in
                    // front for the rows that are off, at the end for the others): whole sectors, and 6 store
                    // instructions per warp instead of 11.  (The store burst of the sampler
                    // holds up every shared-memory and barrier operation of the SM behind it.)
                    constexpr int kRow = kA + 1;
                    static_assert(kRow % 8 == 4, "row = five 32-byte pieces and one 16-byte piece");
                    float rowv[kRow];
#pragma unroll
                    for (int a = 0; a < kA; a++) rowv[a] = logits[a];
                    rowv[kA] = value;
                    float* dst = P.logits_av + (size_t)env * kRow;
                    // (the array itself need only be 16-byte aligned: what counts is the row's address)
                    const bool odd = (reinterpret_cast<uintptr_t>(dst) & 31u) != 0;
                    float4 v4;
                    v4.x = odd ? rowv[0] : rowv[kRow - 4];
                    v4.y = odd ? rowv[1] : rowv[kRow - 3];
                    v4.z = odd ? rowv[2] : rowv[kRow - 2];
                    v4.w = odd ? rowv[3] : rowv[kRow - 1];
                    *reinterpret_cast<float4*>(dst + (odd ? 0 : kRow - 4)) = v4;
#pragma unroll
                    for (int q = 0; q < kRow / 8; q++) {
                        float v8[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) v8[e] = odd ? rowv[8 * q + 4 + e] : rowv[8 * q + e];
                        st_global_v8(dst + 8 * q + (odd ? 4 : 0), v8);
                    }
                }
                float lp;
                const int act = sample_action<kA>(logits, u, &lp);
                if (P.env_actions) P.env_actions[env] = (float)act;
                P.actions[env] = act;
                if (P.logprobs) P.logprobs[env] = lp;
                if (P.values) P.values[env] = value;
            }
            CFX_MARK(11);
        }
    }
    CFX_MARK_FLUSH();
}

// ------------------------------------------------------------------ kernel
// PAIR = false: one CTA per 128-env tile.  PAIR = true: launched as clusters of two CTAs; CTA r
// of a pair owns tile 2 c + r in every respect (records, state, expand, cell, sampler) except
// that the MMA thread of the even CTA issues one 256-row MMA for both tiles and every CTA
// stages only its half of the weight rows.
template <typename T16, bool PAIR, int GAME, int HID>
__global__ void __launch_bounds__(kThreads, 1)
k_policy_fused(const __grid_constant__ Params P) {
    using C = Cfg<PAIR, GAME, HID>;
    CFX_DIMS(HID);
    constexpr int kA = Gm<GAME>::kA;
    // predicates of the deferred probes: MMA thread (weights, operand chunks), workers (operand
    // slot, records, state box, next accumulator)
    CFX_PROBE_DECL(cfx_p_b);
    CFX_PROBE_DECL(cfx_p_a);
    CFX_PROBE_DECL(cfx_p_ae);
    CFX_PROBE_DECL(cfx_p_r);
    CFX_PROBE_DECL(cfx_p_s);
    CFX_PROBE_DECL(cfx_p_g);
    extern __shared__ uint8_t smem_raw[];
    Smem sm;
    sm.base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    sm.template layout<PAIR, GAME, HID>();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    // arrivals per phase on the barriers the MMA thread waits on: both CTAs' workers in a pair
    const uint32_t both = (PAIR && rank == 0) ? 2u : 1u;

    if (tid == 0) {
        auto init = [&](int first, int count, uint32_t arrivals) {
            for (int i = 0; i < count; i++) mbar_init(sm.bar(first + i), arrivals);
        };
        init(B_FULL, C::kNB, 1);   // pair: the even CTA's barrier also counts the odd CTA's bytes
        init(B_EMPTY, C::kNB, 1);
        init(S_FULL, C::kNS, 1);
        init(S_FREE, C::kNS, 1);
        init(ST_READY, C::kNS, 4);
        init(R_FULL, C::kNR, 1);
        init(R_EMPTY, C::kNR, 4);
        init(AEXP_FULL, kAexpSlots, 4 * both);
        init(AEXP_EMPTY, kAexpSlots, 1);
        init(ACC_FULL, 1, 1);
        init(A_KB, kKBlocks, 8 * both);
        init(G_FULL, 1, 1);
        init(G_EMPTY, 1, 8 * both);
        init(H_FULL, 1, 1);
        init(H_EMPTY, 1, 4 * both);
        init(ACC_READ, 1, 8 * both);
        init(REC_DONE, 1, 8);      // full game: every worker warp, after its last chunk
        init(T_FULL, 1, 1);        // classic game: the record buffer, read by both warpgroups
        init(T_EMPTY, 1, 8);
        *sm.abort_flag() = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(smem_u32(sm.tmem_base()), 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(sm.tmem_base()), 512);
            tmem_relinquish();
        }
    }
    if (warp == 3 && lane == 31) {
        prefetch_tensormap(&P.rec_map);
        for (int l = 0; l < P.L; l++) prefetch_tensormap(&P.state_map[l]);
    }
    for (int i = tid; i < kH + kHeadMax; i += kThreads) {
        float v = 0.0f;
        if (i < kH) v = P.params[P.off_b_enc + i];
        else if (i - kH < kA) v = P.params[P.off_b_a + (i - kH)];
        else if (i - kH == kA) v = P.params[P.off_b_v];
        sm.bias()[i] = v;
    }
    tc_fence_before_sync();
    // in a pair the peer's barriers must be initialised before anybody arrives on them
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *sm.tmem_base();
    const uint32_t bar0_cta0 = PAIR ? map_to_cta(sm.bar(0), 0u) : 0u;

    if (warp == 0) {
        if (lane == 0) role_weight_loads<PAIR, GAME, HID>(sm, P, lane, rank, bar0_cta0);
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) role_mma<T16, PAIR, GAME, HID>(sm, P, tmem);
    } else if (warp == 2) {
        if (lane == 0) role_loads<PAIR, GAME, HID>(sm, P);
    } else if (warp == 3) {
        if (lane == 0) role_stores<PAIR, GAME, HID>(sm, P);
    } else {
        role_worker<T16, PAIR, GAME, HID>(sm, P, tmem, warp, lane, bar0_cta0);
    }

    // common exit: every role ends here, also after a timed-out wait.  In a pair neither CTA
    // may release its shared and tensor memory while the peer can still signal or read it.
    __syncwarp();
    tc_fence_before_sync();
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    const uint32_t aborted = *sm.abort_flag();
    if (aborted != 0) {
        if (tid == 0) atomicCAS(P.status, 0u, aborted | ((uint32_t)blockIdx.x << 8));
        // give copies that are still in flight time to land before shared memory is released
        for (int i = 0; i < 64; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        if (PAIR) tmem_dealloc_pair(tmem, 512);
        else tmem_dealloc(tmem, 512);
    }
    // The reference bumps the sampler offset with a one-thread kernel after the step
    // (k_bump_ctr, craftax_full.cu:12085).  Here the last block to finish does it: every block
    // read the counter (in its sampler threads) before it got here.
    if (tid == 0 && P.bump_step) {
        __threadfence();
        if (atomicAdd(P.done_ctr, 1u) == gridDim.x - 1) {
            *P.step_ctr += 1ULL;
            *P.done_ctr = 0u;
        }
    }
}

// Self-test of the bounded wait: one block waits on a barrier on which nothing ever arrives,
// with a limit of a few milliseconds, gives up, and reports through the same status word
// protocol as the forward kernel.  The kernel ends normally; the context stays usable.
constexpr uint32_t kSelftestCode = 0x7E;
__global__ void k_selftest_wait_timeout(uint32_t* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, kSelftestCode, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag != 0) atomicCAS(status, 0u, abort_flag | ((uint32_t)blockIdx.x << 8));
}

}  // namespace fused

int fused_selftest_wait_timeout(unsigned limit_ms, unsigned* status_out) {
    uint32_t* d = nullptr;
    CFX_CUDA(cudaMalloc((void**)&d, sizeof(uint32_t)));
    cudaError_t e = cudaMemset(d, 0, sizeof(uint32_t));
    if (e == cudaSuccess) {
        fused::k_selftest_wait_timeout<<<1, 64>>>(d, (unsigned long long)limit_ms * 1000000ull);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    uint32_t v = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&v, d, sizeof(v), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return cuda_fail(e, "selftest", __FILE__, __LINE__);
    *status_out = v;
    return CFX_OK;
}

// ------------------------------------------------------------------ host side
struct FusedPlan {
    int device, n, H, L, A, precision;
    int game = CFX_GAME_FULL;
    uint8_t* image = nullptr;
    uint32_t* status = nullptr;    // [0] status word, [1] finished-block counter
    float* state = nullptr;
    const float* params = nullptr;
    CUtensorMap state_map[fused::kMaxLayers];
    CUtensorMap w_map[3];          // pair mode: operand image regions (encoder, gates, heads)
    int sm_count = 0;
    int pair = 0;        // 1: launch as clusters of two CTAs (cta_group::2 MMAs)
    int max_pairs = 0;   // co-resident clusters of two
};

bool fused_supported(int H, int L, int A, int precision, int game) {
    const int want_a = game == CFX_GAME_CLASSIC ? fused::Gm<CFX_GAME_CLASSIC>::kA : fused::Gm<CFX_GAME_FULL>::kA;
    // hidden 256 for both games, hidden 128 for the full game
    const bool shape = H == 256 || (H == 128 && game == CFX_GAME_FULL);
    return shape && A == want_a && L >= 1 && L <= fused::kMaxLayers &&
           (precision == CFX_PREC_F16 || precision == CFX_PREC_BF16);
}

// kernel instantiation and its shared-memory size for (operand type, launch mode, game, hidden)
static const void* fused_kernel(int precision, int pair, int game, int H, int* smem) {
    const bool h = precision == CFX_PREC_F16;
#define CFX_K(T, P, G, HID)                                         \
    do {                                                            \
        *smem = fused::Cfg<P, G, HID>::kSmemBytes;                  \
        return (const void*)fused::k_policy_fused<T, P, G, HID>;    \
    } while (0)
#define CFX_K2(P, G, HID)                          \
    do {                                           \
        if (h) CFX_K(__half, P, G, HID);           \
        else CFX_K(__nv_bfloat16, P, G, HID);      \
    } while (0)
    if (game == CFX_GAME_CLASSIC) {
        if (pair) CFX_K2(true, CFX_GAME_CLASSIC, 256);
        CFX_K2(false, CFX_GAME_CLASSIC, 256);
    }
    if (H == 128) {
        if (pair) CFX_K2(true, CFX_GAME_FULL, 128);
        CFX_K2(false, CFX_GAME_FULL, 128);
    }
    if (pair) CFX_K2(true, CFX_GAME_FULL, 256);
    CFX_K2(false, CFX_GAME_FULL, 256);
#undef CFX_K2
#undef CFX_K
}

static size_t fused_image_bytes(int game, int H, int L) {
    if (game == CFX_GAME_CLASSIC) return fused::image_bytes<CFX_GAME_CLASSIC, 256>(L);
    return H == 128 ? fused::image_bytes<CFX_GAME_FULL, 128>(L) : fused::image_bytes<CFX_GAME_FULL, 256>(L);
}

int fused_create(FusedPlan** out, int device, int n, int H, int L, int A, int precision,
                 float* state, int game) {
    if (!fused_supported(H, L, A, precision, game)) {
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
    p->game = game;
    p->state = state;
    p->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaMalloc((void**)&p->image, fused_image_bytes(game, H, L));
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->status, 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(p->status, 0, 2 * sizeof(uint32_t));
    if (e != cudaSuccess) {
        fused_destroy(p);
        return cuda_fail(e, "fused_create alloc", __FILE__, __LINE__);
    }
    for (int l = 0; l < L; l++) {
        if (!make_tmap_2d(&p->state_map[l], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                          state + (size_t)l * n * H, (uint64_t)n, (uint64_t)H, (uint64_t)H * 4,
                          fused::kTile, fused::kHalfUnits, CU_TENSOR_MAP_SWIZZLE_128B)) {
            fused_destroy(p);
            set_error("fused_create: cuTensorMapEncodeTiled failed for the state");
            return CFX_ERR_CUDA;
        }
    }
    for (int pr = 0; pr < 2 && e == cudaSuccess; pr++) {
        int smem = 0;
        const void* k = fused_kernel(precision, pr, game, H, &smem);
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    if (e != cudaSuccess) {
        fused_destroy(p);
        return cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__);
    }
    // CTA pairs are the default (CFX_FUSED_PAIR=0 selects one CTA per tile); they need two
    // co-resident CTAs per cluster, otherwise the single-CTA kernel is used
    const char* pe = getenv("CFX_FUSED_PAIR");
    if (pe == nullptr || atoi(pe) != 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)(p->sm_count / 2));
        cfg.blockDim = dim3(fused::kThreads);
        int smem = 0;
        const void* kpair = fused_kernel(precision, 1, game, H, &smem);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute at;
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
        cfg.attrs = &at; cfg.numAttrs = 1;
        int nc = 0;
        if (cudaOccupancyMaxActiveClusters(&nc, kpair, &cfg) == cudaSuccess && nc > 0) {
            p->pair = 1;
            p->max_pairs = nc;
        } else {
            cudaGetLastError();
        }
    }
    memset(p->w_map, 0, sizeof(p->w_map));
    if (p->pair) {
        // The operand image seen as rows of 64 16-bit values (128 bytes), one tensor per region;
        // a box is what ONE CTA of a pair copies of a stage: half of a two-chunk encoder stage,
        // half of a two-K-block gate stage, half of the head stage.  The image is already
        // swizzled, so the copies are not.
        const bool classic = game == CFX_GAME_CLASSIC;
        const int kblocks = H / 64;
        const int enc_chunks = classic ? fused::Gm<CFX_GAME_CLASSIC>::kEncBlocks : fused::Gm<CFX_GAME_FULL>::kEncBlocks;
        const int head_pair = classic ? fused::Gm<CFX_GAME_CLASSIC>::kHeadPair : fused::Gm<CFX_GAME_FULL>::kHeadPair;
        const uint64_t rows[3] = {(uint64_t)enc_chunks * H, (uint64_t)L * (H / 64) * kblocks * 192,
                                  (uint64_t)kblocks * head_pair};
        const uint32_t box[3] = {(uint32_t)H, 192u, (uint32_t)(kblocks * head_pair / 2)};
        uint8_t* base = p->image;
        for (int r = 0; r < 3; r++) {
            if (!make_tmap_2d(&p->w_map[r], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, rows[r], 64, 128, box[r], 64,
                              CU_TENSOR_MAP_SWIZZLE_NONE)) {
                fused_destroy(p);
                set_error("fused_create: cuTensorMapEncodeTiled failed for the operand image");
                return CFX_ERR_CUDA;
            }
            base += rows[r] * 128;
        }
    }
    *out = p;
    return CFX_OK;
}

int fused_refresh(FusedPlan* p, const float* params, cudaStream_t st) {
    p->params = params;
    const bool classic = p->game == CFX_GAME_CLASSIC;
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A, classic ? kClassicObs : kObs);
    const size_t total = fused_image_bytes(p->game, p->H, p->L) / 2;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    const bool h = p->precision == CFX_PREC_F16;
#define CFX_PACK(T, G, HID) fused::k_pack_image<T, G, HID><<<blocks, 256, 0, st>>>(params, p->image, p->L, o.w_gru, o.w_a, o.w_v, p->pair)
    if (classic) { if (h) CFX_PACK(__half, CFX_GAME_CLASSIC, 256); else CFX_PACK(__nv_bfloat16, CFX_GAME_CLASSIC, 256); }
    else if (p->H == 128) { if (h) CFX_PACK(__half, CFX_GAME_FULL, 128); else CFX_PACK(__nv_bfloat16, CFX_GAME_FULL, 128); }
    else { if (h) CFX_PACK(__half, CFX_GAME_FULL, 256); else CFX_PACK(__nv_bfloat16, CFX_GAME_FULL, 256); }
#undef CFX_PACK
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

int fused_forward(FusedPlan* p, const FusedArgs& a, cudaStream_t st, int* launches) {
    if (a.r_state != nullptr && ((uintptr_t)a.r_state & 15) != 0) {
        set_error("fused forward: r_state must be 16-byte aligned");
        return CFX_ERR_INVALID;
    }
    if (a.logits_av != nullptr && ((uintptr_t)a.logits_av & 15) != 0) {
        set_error("fused forward: logits_av must be 16-byte aligned");
        return CFX_ERR_INVALID;
    }
    fused::Params P;
    const bool classic = p->game == CFX_GAME_CLASSIC;
    // records as rows of four: full game uint8 [n/4][3984], boxes of 32 rows x 80 bytes;
    // classic uint32 [n/4][148] (592 bytes), one box of 32 rows x 148 words per tile
    const bool ok_map = classic
        ? make_tmap_2d(&P.rec_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, (void*)a.records, (uint64_t)p->n / 4,
                       (uint64_t)kClassicRec, (uint64_t)kClassicRec * 4, 32, kClassicRec, CU_TENSOR_MAP_SWIZZLE_NONE)
        : make_tmap_2d(&P.rec_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (void*)a.records, (uint64_t)p->n / 4,
                       (uint64_t)kRec * 4, (uint64_t)kRec * 4, 32, 80, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok_map) {
        set_error("fused forward: cuTensorMapEncodeTiled failed for the records");
        return CFX_ERR_CUDA;
    }
    for (int l = 0; l < p->L; l++) P.state_map[l] = p->state_map[l];
    for (int r = 0; r < 3; r++) P.w_map[r] = p->w_map[r];
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A, classic ? kClassicObs : kObs);
    P.records = a.records;
    P.rec_bytes = classic ? kClassicRec : kRec;
    P.state = a.state;
    P.image = p->image;
    P.params = p->params;
    P.prev_terminals = a.prev_terminals;
    P.uniforms = a.uniforms;
    P.env_actions = a.env_actions;
    P.actions = a.actions;
    P.logprobs = a.logprobs;
    P.values = a.values;
    P.logits_av = a.logits_av;
    P.r_state = a.r_state;
    P.r_state_bf16 = a.r_state_bf16;
    P.step_ctr = a.step_ctr;
    P.status = p->status;
    P.done_ctr = p->status + 1;
    P.bump_step = a.bump_step;
    P.seed = a.seed;
    P.env_offset = a.env_offset;
    P.n = p->n;
    P.L = p->L;
    const int all_tiles = (p->n + fused::kTile - 1) / fused::kTile;
    P.tile_begin = a.tile_end > 0 ? a.tile_begin : 0;
    P.num_tiles = a.tile_end > 0 ? a.tile_end : all_tiles;
    // a CTA pair works on tiles 2c, 2c + 1: a slice must start at an even tile, and only the
    // slice that ends the batch may hold an odd number of tiles (its filler tile lies beyond n)
    if (P.tile_begin < 0 || P.num_tiles > all_tiles || P.tile_begin >= P.num_tiles || (P.tile_begin & 1) ||
        ((P.num_tiles & 1) && P.num_tiles != all_tiles)) {
        set_error("fused forward: bad tile range [%d, %d) of %d", P.tile_begin, P.num_tiles, all_tiles);
        return CFX_ERR_INVALID;
    }
    const int range_tiles = P.num_tiles - P.tile_begin;
    P.off_b_enc = o.b_enc;
    P.off_b_a = o.b_a;
    P.off_b_v = o.b_v;
    int smem = 0;
    const void* kern = fused_kernel(p->precision, p->pair, p->game, p->H, &smem);
    void* kargs[1] = {(void*)&P};
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(fused::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at;
    if (p->pair) {
        const int pairs = (range_tiles + 1) / 2;
        P.num_tiles_loop = P.tile_begin + 2 * pairs;
        cfg.gridDim = dim3(2u * (unsigned)(pairs < p->max_pairs ? pairs : p->max_pairs));
        at.id = cudaLaunchAttributeClusterDimension;
        at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
        cfg.attrs = &at; cfg.numAttrs = 1;
    } else {
        P.num_tiles_loop = P.num_tiles;
        cfg.gridDim = dim3((unsigned)(range_tiles < p->sm_count ? range_tiles : p->sm_count));
    }
    CFX_CUDA(cudaLaunchKernelExC(&cfg, kern, kargs));
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
