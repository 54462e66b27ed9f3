// Record write: env state -> 996-byte compact records (reference k_record_obs /
// cf_record_env_warp, craftax_full.cu:9180-9297; scalar tail :2429-2487).
//
// The reference gives every env a warp and lets lane 0 walk the mob slots and compute the 51
// tail scalars; every one of its ~110 scalar loads then fetches 4 bytes of a sector on its own,
// one after the other.  Here a block of four warps owns 32 consecutive envs and works in two
// phases:
//   1. lane per env: the ~50 SoA fields and the 14 mob slots of the player's level (type, mask,
//      position, light at the position) are loaded by lane e for env e, so that a warp's loads
//      of a field are one 128-byte line and all loads of a lane are independent; each warp takes
//      a quarter of the fields; they leave the 51 tail floats, the visible mobs (an earlier slot
//      of a class that a later slot covers is dropped) and (level, top, left) in shared memory;
//   2. warp per env (8 envs per warp, the next env's loads in flight while one is stored): the
//      99 view cells, 8 bytes each from three byte maps, go out as coalesced 8-byte stores,
//      then one lane per visible mob stores its byte, then the tail goes out as coalesced
//      4-byte stores from shared memory.
// The bytes are the reference's: the same predicates, the same "last slot of a class wins a
// cell" order, the same float expressions (sqrtf(x) * 0.1f, x * 0.1f, x * 0.5f, x * 0.25f; no
// fused multiply-add can form).  HBM traffic per env: 996 B written, 27 map sectors (9 rows of
// 11 bytes in three maps) and ~100 SoA words read.
#include <cuda_runtime.h>

#include <cstddef>

#include "cfx_common.cuh"

namespace cfx {
namespace record {

constexpr int kRows = 9, kCols = 11, kCells = kRows * kCols;   // view around the player
constexpr int kMapSize = 48, kLevels = 9, kMobTypes = 8, kClasses = 5, kSlots = 3;
constexpr int kMobs = kClasses * kSlots;                       // slot 2 of class 2 is never used
constexpr int kLit = 12;                                       // light_map > 12 = visible
constexpr int kKilledToClear = 8;
constexpr int kBlockEnvs = 32, kBlockThreads = 128;

struct Params {
    cfx_env_view v;
    uint8_t* records;
    const uint8_t* skip;
    const uint8_t* list;
    int list_stride;
    const int* count_dev;
    int n;
};
struct Shared {
    float tail[kBlockEnvs][kTail];       // odd row length: conflict-free thread-per-env writes
    uint32_t mobs[kBlockEnvs][kMobs];
    int32_t level[kBlockEnvs], top[kBlockEnvs], left[kBlockEnvs], env[kBlockEnvs];   // env < 0: nothing to write
};

// craftax_wg_jax_index (:1963-1975): negative indices wrap once, then clamp
__device__ __forceinline__ int jax_index(int i, int size) {
    if (i < 0) i += size;
    if (i < 0) return 0;
    return i >= size ? size - 1 : i;
}
template <typename T>
__device__ __forceinline__ T soa(const T* f, int elem, int n, int e) {
    return f[(size_t)elem * (size_t)n + (size_t)e];
}
// flat index of (class, level, slot) in the mob fields (CFM, :715)
__device__ __forceinline__ int mob_index(int c, int level, int i) { return (c * kLevels + level) * kSlots + i; }

// phase 1: everything of env e that does not depend on the cell.  Lane t of EVERY warp of the
// block works on env t of the block; warp `part` takes a quarter of the work:
//   part 0: tail scalars 0-25        part 1: tail scalars 26-49
//   part 2: mob classes 0-2 + the boss flag (tail scalar 50)        part 3: mob classes 3-4
__device__ __forceinline__ void gather_env(const cfx_env_view& V, int e, int t, int part, Shared& S) {
    const int n = V.num_envs;
    const int level = soa(V.player_level, 0, n, e);
    float* o = S.tail[t];
    int k = 0;
    auto sq10 = [&](const int32_t* f, int i) { o[k++] = sqrtf((float)soa(f, i, n, e)) * (1.0f / 10.0f); };
    auto mul = [&](const int32_t* f, int i, float m) { o[k++] = (float)soa(f, i, n, e) * m; };
    auto flag = [&](bool b) { o[k++] = b ? 1.0f : 0.0f; };
    // the 51 scalars in the order of craftax_encode_scalar_observation_tail_at (:2429-2487)
    if (part == 0) {
        sq10(V.inv_wood, 0); sq10(V.inv_stone, 0); sq10(V.inv_coal, 0); sq10(V.inv_iron, 0);
        sq10(V.inv_diamond, 0); sq10(V.inv_sapphire, 0); sq10(V.inv_ruby, 0); sq10(V.inv_sapling, 0);
        sq10(V.inv_torches, 0); sq10(V.inv_arrows, 0);
        mul(V.inv_books, 0, 1.0f / 2.0f);
        mul(V.inv_pickaxe, 0, 1.0f / 4.0f);
        mul(V.inv_sword, 0, 1.0f / 4.0f);
        o[k++] = (float)soa(V.sword_enchantment, 0, n, e);
        o[k++] = (float)soa(V.bow_enchantment, 0, n, e);
        o[k++] = (float)soa(V.inv_bow, 0, n, e);
#pragma unroll
        for (int i = 0; i < 6; i++) sq10(V.inv_potions, i);
        o[k++] = soa(V.player_health, 0, n, e) * (1.0f / 10.0f);
        mul(V.player_food, 0, 1.0f / 10.0f); mul(V.player_drink, 0, 1.0f / 10.0f);
        mul(V.player_energy, 0, 1.0f / 10.0f);   // scalar 25
        return;
    }
    if (part == 1) {
        k = 26;
        mul(V.player_mana, 0, 1.0f / 10.0f);
        mul(V.player_xp, 0, 1.0f / 10.0f); mul(V.player_dexterity, 0, 1.0f / 10.0f);
        mul(V.player_strength, 0, 1.0f / 10.0f); mul(V.player_intelligence, 0, 1.0f / 10.0f);
        const int direction_index = soa(V.player_direction, 0, n, e) - 1;
#pragma unroll
        for (int i = 0; i < 4; i++) flag(i == direction_index);
#pragma unroll
        for (int i = 0; i < 4; i++) mul(V.inv_armour, i, 1.0f / 2.0f);
#pragma unroll
        for (int i = 0; i < 4; i++) o[k++] = (float)soa(V.armour_enchantments, i, n, e);
        o[k++] = soa(V.light_level, 0, n, e);
        flag(soa(V.is_sleeping, 0, n, e) != 0);
        flag(soa(V.is_resting, 0, n, e) != 0);
        flag(soa(V.learned_spells, 0, n, e) != 0);
        flag(soa(V.learned_spells, 1, n, e) != 0);
        mul(V.player_level, 0, 1.0f / 10.0f);
        flag((unsigned)level < (unsigned)kLevels && soa(V.monsters_killed, level, n, e) >= kKilledToClear);   // scalar 49
        return;
    }
    // visible mobs of the player's level, class-major, slot-minor (:9195-9236):
    // packed = valid | cell << 8 | channel << 4 | value
    const int mob_level = jax_index(level, kLevels);
    const int top = soa(V.player_position, 0, n, e) - kRows / 2;
    const int left = soa(V.player_position, 1, n, e) - kCols / 2;
    const uint8_t* light = V.state_base + (size_t)e * V.state_stride + V.light_map_offset +
                           (size_t)mob_level * kMapSize * kMapSize;
    const int c0 = part == 2 ? 0 : 3, c1 = part == 2 ? 3 : kClasses;
    bool melee_or_ranged = false;
    for (int c = c0; c < c1; c++) {
        uint32_t pk[kSlots];
#pragma unroll
        for (int i = 0; i < kSlots; i++) {
            pk[i] = 0;
            if (i < (c == 2 ? 2 : 3)) {
                const int idx = mob_index(c, mob_level, i);
                const int type_id = soa(V.mob_type_id, idx, n, e);
                const bool mask = soa(V.mob_mask, idx, n, e) != 0;
                if (c == 0 || c == 2) melee_or_ranged = melee_or_ranged || mask;
                const int mr = soa(V.mob_position, idx * 2, n, e), mc = soa(V.mob_position, idx * 2 + 1, n, e);
                const int lr = mr - top, lc = mc - left;
                if (type_id >= 0 && type_id < kMobTypes && mask && lr >= 0 && lr < kRows && lc >= 0 && lc < kCols &&
                    mr >= 0 && mr < kMapSize && mc >= 0 && mc < kMapSize && light[mr * kMapSize + mc] > kLit)
                    pk[i] = 0x80000000u | (uint32_t)(lr * kCols + lc) << 8 | (uint32_t)(3 + c) << 4 |
                            (uint32_t)(type_id + 1);
            }
        }
        // "last slot wins": a later slot of the class on the same cell replaces an earlier one
        // (:9222-9231); the earlier one is dropped here, so the stores of phase 2 need no order
#pragma unroll
        for (int i = 0; i < kSlots - 1; i++)
#pragma unroll
            for (int i2 = i + 1; i2 < kSlots; i2++)
                if ((pk[i] & pk[i2] & 0x80000000u) && ((pk[i] ^ pk[i2]) & 0xFF00u) == 0) pk[i] = 0;
#pragma unroll
        for (int i = 0; i < kSlots; i++) S.mobs[t][c * kSlots + i] = pk[i];
    }
    if (part == 2) {
        // craftax_wg_is_boss_vulnerable (:1988-2003): no melee and no ranged mob alive on the level
        o[kTail - 1] = !melee_or_ranged && soa(V.boss_timesteps_to_spawn_this_round, 0, n, e) <= 0 ? 1.0f : 0.0f;
    } else {
        S.level[t] = level; S.top[t] = top; S.left[t] = left;
    }
}

// phase 2: the cells of one env.  The three byte loads per cell of all four rounds are issued
// at once (load_cells); the caller holds them in registers while it stores the previous env.
struct Cells { uint32_t l[4], b[4], it[4]; };
__device__ __forceinline__ void load_cells(const cfx_env_view& V, const Shared& S, int t, int lane, Cells& c) {
    const int e = S.env[t];
    if (e < 0) return;
    const int level = S.level[t], top = S.top[t], left = S.left[t];
    const uint8_t* blk = V.state_base + (size_t)e * V.state_stride + (size_t)level * kMapSize * kMapSize;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int cell = lane + 32 * r;
        const int wr = top + cell / kCols, wc = left + cell % kCols;
        // (a level outside [0, 9) never comes out of the env; the reference would read outside
        // its maps there, here such an env gets unlit cells)
        const bool in = cell < kCells && wr >= 0 && wr < kMapSize && wc >= 0 && wc < kMapSize &&
                        (unsigned)level < (unsigned)kLevels;
        const int o = in ? wr * kMapSize + wc : 0;
        c.l[r] = in ? blk[V.light_map_offset + o] : 0u;
        c.b[r] = in ? blk[V.map_offset + o] : 0u;
        c.it[r] = in ? blk[V.item_map_offset + o] : 0u;
    }
}
// map cells: 8 bytes each {block, item + 1, lit, five mob classes}  (:9241-9269), then the tail
__device__ __forceinline__ void store_env(const Params& P, const Shared& S, int t, int lane, const Cells& c) {
    const int e = S.env[t];
    if (e < 0) return;
    uint8_t* rec = P.records + (size_t)e * kRec;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int cell = lane + 32 * r;
        if (cell < kCells) {
            const uint32_t w0 = c.l[r] > (uint32_t)kLit ? (c.b[r] | ((c.it[r] + 1u) & 0xFFu) << 8 | 1u << 16) : 0u;
            uint32_t* dst = reinterpret_cast<uint32_t*>(rec + (size_t)cell * 8);   // 4-byte aligned (996 = 4 x 249)
            dst[0] = w0;
            dst[1] = 0u;
        }
    }
    __syncwarp();   // the mob bytes land on cells other lanes have just written
    if (lane < kMobs) {
        const uint32_t pk = S.mobs[t][lane];
        if (pk & 0x80000000u) rec[(size_t)((pk >> 8) & 0xFFu) * 8 + ((pk >> 4) & 0xFu)] = (uint8_t)(pk & 0xFu);
    }
    for (int j = lane; j < kTail; j += 32) *reinterpret_cast<float*>(rec + kMap + 4 * j) = S.tail[t][j];
}
// warp `warp` writes envs warp, warp + 4, ... of the block, loading one env ahead
__device__ __forceinline__ void write_envs(const Params& P, const Shared& S, int warp, int lane) {
    constexpr int kWarps = kBlockThreads / 32;
    Cells cur, nxt;
    load_cells(P.v, S, warp, lane, cur);
    for (int k = warp; k < kBlockEnvs; k += kWarps) {
        if (k + kWarps < kBlockEnvs) load_cells(P.v, S, k + kWarps, lane, nxt);
        store_env(P, S, k, lane, cur);
        if (k + kWarps < kBlockEnvs) cur = nxt;
    }
}

__global__ void __launch_bounds__(kBlockThreads) k_record_rows(const __grid_constant__ Params P) {
    __shared__ Shared S;   // 9 KB
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int e = blockIdx.x * kBlockEnvs + lane;
    const bool live = e < P.n && (P.skip == nullptr || P.skip[e] == 0);
    if (live) gather_env(P.v, e, lane, warp, S);
    if (warp == 0) S.env[lane] = live ? e : -1;
    __syncthreads();
    write_envs(P, S, warp, lane);
}

// the envs named by a device-side list (first int32 of every entry), 32 entries per block pass
__global__ void __launch_bounds__(kBlockThreads) k_record_rows_list(const __grid_constant__ Params P) {
    __shared__ Shared S;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int count = *P.count_dev;
    for (int base = blockIdx.x * kBlockEnvs; base < count; base += (int)gridDim.x * kBlockEnvs) {
        int e = -1;
        if (base + lane < count) e = *reinterpret_cast<const int32_t*>(P.list + (size_t)(base + lane) * P.list_stride);
        const bool live = e >= 0 && e < P.v.num_envs;
        if (live) gather_env(P.v, e, lane, warp, S);
        if (warp == 0) S.env[lane] = live ? e : -1;
        __syncthreads();
        write_envs(P, S, warp, lane);
        __syncthreads();
    }
}

static int make_params(const char* who, const cfx_env_view* view, uint8_t* records, Params* P) {
    CFX_REQUIRE(view != nullptr && records != nullptr, "%s: bad argument", who);
    CFX_REQUIRE(view->num_envs > 0 && view->state_base != nullptr && view->state_stride > 0,
                "%s: the view has no envs or no state block", who);
    CFX_REQUIRE(((uintptr_t)records & 3) == 0, "%s: records must be 4-byte aligned", who);
    // every field pointer of the view sits between player_position and mob_type_id
    const void* const* first = reinterpret_cast<const void* const*>(&view->player_position);
    const void* const* last = reinterpret_cast<const void* const*>(&view->mob_type_id);
    for (const void* const* q = first; q <= last; q++)
        CFX_REQUIRE(*q != nullptr, "%s: field pointer %d of the view is NULL", who, (int)(q - first));
    P->v = *view;
    P->records = records;
    P->skip = nullptr; P->list = nullptr; P->list_stride = 0; P->count_dev = nullptr;
    P->n = view->num_envs;
    return CFX_OK;
}

static_assert(sizeof(Shared) <= 48 * 1024, "static shared memory");
static_assert(offsetof(cfx_env_view, mob_type_id) - offsetof(cfx_env_view, player_position) == 39 * sizeof(void*),
              "the field pointers of cfx_env_view are contiguous (make_params walks them)");


// ------------------------------------------------------------------ classic game
// record_obs_kernel (craftax_classic.cu:1884-1890) gives every env a thread that writes its 148
// bytes one by one: 148 store instructions per warp, each touching 32 different records.  Here a
// block gathers the records of 128 consecutive envs in shared memory, thread per env (the SoA
// loads of a warp are contiguous), and writes the 18,944 contiguous bytes out as coalesced words.
constexpr int kClRows = 7, kClCols = 9, kClCells = kClRows * kClCols, kClMap = 64, kClRowBytes = 32;
constexpr int kClInv = 12, kClOutOfBounds = 1, kClBlockEnvs = 128;
static_assert(2 * kClCells + kClInv + 6 + 4 == kClassicRec, "classic record layout");

__global__ void __launch_bounds__(kClBlockEnvs) k_classic_record_rows(const __grid_constant__ cfx_classic_env_view V,
                                                                     uint8_t* __restrict__ records, int n_envs) {
    __shared__ __align__(16) uint8_t srec[kClBlockEnvs * kClassicRec];
    const int t = threadIdx.x;
    const int e0 = blockIdx.x * kClBlockEnvs, e = e0 + t;
    const int n = V.num_envs;
    if (e < n_envs) {
        uint8_t* o = srec + t * kClassicRec;
        const int pr = V.player_r[e], pc = V.player_c[e];
        const uint8_t* map = V.map_packed + (size_t)e * V.map_stride;
        // view rows: blocks (a nibble per map column; 1 outside the map), mob bytes cleared  (:1061-1100)
#pragma unroll
        for (int r = 0; r < kClRows; r++) {
            const int mr = pr - 3 + r;
            const bool row_in = mr >= 0 && mr < kClMap;
#pragma unroll
            for (int c = 0; c < kClCols; c++) {
                const int mc = pc - 4 + c;
                uint8_t blk = kClOutOfBounds;
                if (row_in && mc >= 0 && mc < kClMap) {
                    const uint8_t b = map[mr * kClRowBytes + (mc >> 1)];
                    blk = (mc & 1) ? (b >> 4) : (b & 0x0F);
                }
                o[r * kClCols + c] = blk;
                o[kClCells + r * kClCols + c] = 0;
            }
        }
        // mobs inside the view set their bit  (:1102-1125)
        auto stamp = [&](const int16_t* rr, const int16_t* cc, const uint8_t* mask, int slots, uint8_t bit) {
            for (int i = 0; i < slots; i++) {
                if (!mask[(size_t)i * n + e]) continue;
                const int dr = rr[(size_t)i * n + e] - pr, dc = cc[(size_t)i * n + e] - pc;
                if (dr < -3 || dr > 3 || dc < -4 || dc > 4) continue;
                o[kClCells + (dr + 3) * kClCols + (dc + 4)] |= bit;
            }
        };
        stamp(V.zombie_r, V.zombie_c, V.zombie_mask, 3, 1);
        stamp(V.cow_r, V.cow_c, V.cow_mask, 3, 2);
        stamp(V.skel_r, V.skel_c, V.skel_mask, 2, 4);
        stamp(V.arrow_r, V.arrow_c, V.arrow_mask, 3, 8);
        // inventory, intrinsics, direction, sleeping, light  (:1590-1603)
        int idx = 2 * kClCells;
#pragma unroll
        for (int i = 0; i < kClInv; i++) o[idx++] = (uint8_t)V.inv[(size_t)i * n + e];
        o[idx++] = (uint8_t)V.health[e];
        o[idx++] = (uint8_t)V.food[e];
        o[idx++] = (uint8_t)V.drink[e];
        o[idx++] = (uint8_t)V.energy[e];
        o[idx++] = (uint8_t)V.player_dir[e];
        o[idx++] = V.is_sleeping[e] ? 1 : 0;
        const uint32_t light = __float_as_uint(V.light_level[e]);
        o[idx++] = (uint8_t)light; o[idx++] = (uint8_t)(light >> 8);
        o[idx++] = (uint8_t)(light >> 16); o[idx++] = (uint8_t)(light >> 24);
    }
    __syncthreads();
    // the block's records are contiguous in global memory: 37 words per env
    const int envs = min(kClBlockEnvs, n_envs - e0);
    const int words = envs * (kClassicRec / 4);
    uint32_t* dst = reinterpret_cast<uint32_t*>(records + (size_t)e0 * kClassicRec);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(srec);
    for (int w = t; w < words; w += kClBlockEnvs) dst[w] = src[w];
}

}  // namespace record
}  // namespace cfx

using namespace cfx;

extern "C" int cfx_record_obs(int device, const cfx_env_view* view, uint8_t* records, int n, const uint8_t* skip,
                              void* stream) {
    record::Params P;
    int rc = record::make_params("cfx_record_obs", view, records, &P);
    if (rc != CFX_OK) return rc;
    CFX_REQUIRE(n > 0 && n <= view->num_envs, "cfx_record_obs: n=%d outside (0, num_envs=%d]", n, view->num_envs);
    CFX_GUARD(device);
    P.n = n;
    P.skip = skip;
    const unsigned blocks = (unsigned)((n + record::kBlockEnvs - 1) / record::kBlockEnvs);
    record::k_record_rows<<<blocks, record::kBlockThreads, 0, (cudaStream_t)stream>>>(P);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

extern "C" int cfx_record_obs_list(int device, const cfx_env_view* view, uint8_t* records, const void* list,
                                   int list_stride, const int* count_dev, void* stream) {
    record::Params P;
    int rc = record::make_params("cfx_record_obs_list", view, records, &P);
    if (rc != CFX_OK) return rc;
    CFX_REQUIRE(list != nullptr && count_dev != nullptr && list_stride >= 4 && list_stride % 4 == 0,
                "cfx_record_obs_list: bad list");
    CFX_GUARD(device);
    P.list = (const uint8_t*)list;
    P.list_stride = list_stride;
    P.count_dev = count_dev;
    // the count is on the device: a fixed grid walks the list (the reference uses at most
    // 128 blocks of 8 warps for its list pass, :11941)
    int blocks = (view->num_envs + record::kBlockEnvs - 1) / record::kBlockEnvs;
    if (blocks > 592) blocks = 592;
    record::k_record_rows_list<<<blocks, record::kBlockThreads, 0, (cudaStream_t)stream>>>(P);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}

extern "C" int cfx_classic_record_obs(int device, const cfx_classic_env_view* view, uint8_t* records, int n,
                                      void* stream) {
    CFX_REQUIRE(view != nullptr && records != nullptr, "cfx_classic_record_obs: bad argument");
    CFX_REQUIRE(view->num_envs > 0 && n > 0 && n <= view->num_envs,
                "cfx_classic_record_obs: n=%d outside (0, num_envs=%d]", n, view->num_envs);
    CFX_REQUIRE(((uintptr_t)records & 3) == 0, "cfx_classic_record_obs: records must be 4-byte aligned");
    CFX_REQUIRE(view->map_packed != nullptr && view->map_stride >= 64 * 32,
                "cfx_classic_record_obs: the view has no packed map");
    // every field pointer of the view sits between player_r and light_level
    const void* const* first = reinterpret_cast<const void* const*>(&view->player_r);
    const void* const* last = reinterpret_cast<const void* const*>(&view->light_level);
    for (const void* const* q = first; q <= last; q++)
        CFX_REQUIRE(*q != nullptr, "cfx_classic_record_obs: field pointer %d of the view is NULL", (int)(q - first));
    CFX_GUARD(device);
    const unsigned blocks = (unsigned)((n + record::kClBlockEnvs - 1) / record::kClBlockEnvs);
    record::k_classic_record_rows<<<blocks, record::kClBlockEnvs, 0, (cudaStream_t)stream>>>(*view, records, n);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}
