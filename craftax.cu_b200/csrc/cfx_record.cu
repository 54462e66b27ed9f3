// Record write: env state -> 996-byte compact records (reference k_record_obs /
// cf_record_env_warp, craftax_full.cu:9180-9297; scalar tail :2429-2487).
//
// The reference gives every env a warp and lets lane 0 walk the mob slots and compute the 51
// tail scalars; every one of its ~110 scalar loads then fetches 4 bytes of a sector on its own,
// one after the other.  Here a block of four warps owns 32 consecutive envs and works in two
// phases:
//   1. thread per env (one warp): the ~50 SoA fields and the 14 mob slots of the player's level
//      (type, mask, position, light at the position) are loaded by thread e for env e, so that
//      the warp's loads of a field are one 128-byte line and all loads of a thread are
//      independent; the thread leaves the 51 tail floats, the visible mobs (an earlier slot of a
//      class that a later slot covers is dropped) and (level, top, left) in shared memory;
//   2. warp per env (8 envs per warp): the 99 view cells, 8 bytes each from three byte maps, go
//      out as coalesced 8-byte stores, then one lane per visible mob stores its byte, then the
//      tail goes out as coalesced 4-byte stores from shared memory.
// The bytes are the reference's: the same predicates, the same "last slot of a class wins a
// cell" order, the same float expressions (sqrtf(x) * 0.1f, x * 0.1f, x * 0.5f, x * 0.25f; no
// fused multiply-add can form).  HBM traffic per env: 996 B written, 27 map sectors (9 rows of
// 11 bytes in three maps) and ~100 SoA words read.
#include <cuda_runtime.h>

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

// phase 1: everything of env e that does not depend on the cell
__device__ __forceinline__ void gather_env(const cfx_env_view& V, int e, int t, Shared& S) {
    const int n = V.num_envs;
    const int level = soa(V.player_level, 0, n, e);
    const int mob_level = jax_index(level, kLevels);
    const int top = soa(V.player_position, 0, n, e) - kRows / 2;
    const int left = soa(V.player_position, 1, n, e) - kCols / 2;
    S.level[t] = level; S.top[t] = top; S.left[t] = left; S.env[t] = e;
    const uint8_t* light = V.state_base + (size_t)e * V.state_stride + V.light_map_offset +
                           (size_t)mob_level * kMapSize * kMapSize;

    // visible mobs of the player's level, class-major, slot-minor (:9195-9236):
    // packed = valid | cell << 8 | channel << 4 | value
    bool melee_or_ranged = false;
#pragma unroll
    for (int m = 0; m < kMobs; m++) {
        const int c = m / kSlots, i = m % kSlots;
        uint32_t pk = 0;
        if (i < (c == 2 ? 2 : 3)) {
            const int idx = mob_index(c, mob_level, i);
            const int type_id = soa(V.mob_type_id, idx, n, e);
            const bool mask = soa(V.mob_mask, idx, n, e) != 0;
            if (c == 0 || c == 2) melee_or_ranged = melee_or_ranged || mask;
            const int mr = soa(V.mob_position, idx * 2, n, e), mc = soa(V.mob_position, idx * 2 + 1, n, e);
            const int lr = mr - top, lc = mc - left;
            if (type_id >= 0 && type_id < kMobTypes && mask && lr >= 0 && lr < kRows && lc >= 0 && lc < kCols &&
                mr >= 0 && mr < kMapSize && mc >= 0 && mc < kMapSize && light[mr * kMapSize + mc] > kLit)
                pk = 0x80000000u | (uint32_t)(lr * kCols + lc) << 8 | (uint32_t)(3 + c) << 4 | (uint32_t)(type_id + 1);
        }
        S.mobs[t][m] = pk;
    }
    // "last slot wins": within a class a later slot on the same cell replaces an earlier one
    // (:9222-9231), so the earlier one is dropped here and the stores of phase 2 need no order
#pragma unroll
    for (int c = 0; c < kClasses; c++)
#pragma unroll
        for (int i = 0; i < kSlots - 1; i++)
#pragma unroll
            for (int i2 = i + 1; i2 < kSlots; i2++) {
                const uint32_t a = S.mobs[t][c * kSlots + i], b = S.mobs[t][c * kSlots + i2];
                if ((a & b & 0x80000000u) && ((a ^ b) & 0xFF00u) == 0) S.mobs[t][c * kSlots + i] = 0;
            }

    // the 51 scalars in the order of craftax_encode_scalar_observation_tail_at (:2429-2487)
    float* o = S.tail[t];
    int k = 0;
    auto sq10 = [&](const int32_t* f, int i) { o[k++] = sqrtf((float)soa(f, i, n, e)) * (1.0f / 10.0f); };
    auto mul = [&](const int32_t* f, int i, float m) { o[k++] = (float)soa(f, i, n, e) * m; };
    auto flag = [&](bool b) { o[k++] = b ? 1.0f : 0.0f; };
    sq10(V.inv_wood, 0); sq10(V.inv_stone, 0); sq10(V.inv_coal, 0); sq10(V.inv_iron, 0); sq10(V.inv_diamond, 0);
    sq10(V.inv_sapphire, 0); sq10(V.inv_ruby, 0); sq10(V.inv_sapling, 0); sq10(V.inv_torches, 0); sq10(V.inv_arrows, 0);
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
    mul(V.player_energy, 0, 1.0f / 10.0f); mul(V.player_mana, 0, 1.0f / 10.0f);
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
    flag(soa(V.monsters_killed, level, n, e) >= kKilledToClear);
    // craftax_wg_is_boss_vulnerable (:1988-2003): no melee and no ranged mob alive on the level
    flag(!melee_or_ranged && soa(V.boss_timesteps_to_spawn_this_round, 0, n, e) <= 0);
}

// phase 2: one warp writes the record of the env that thread t gathered
__device__ __forceinline__ void write_env(const Params& P, const Shared& S, int t, int lane) {
    const int e = S.env[t];
    if (e < 0) return;
    const cfx_env_view& V = P.v;
    uint8_t* rec = P.records + (size_t)e * kRec;
    const int level = S.level[t], top = S.top[t], left = S.left[t];
    const uint8_t* blk = V.state_base + (size_t)e * V.state_stride + (size_t)level * kMapSize * kMapSize;
    const uint8_t* map = blk + V.map_offset;
    const uint8_t* item = blk + V.item_map_offset;
    const uint8_t* lit = blk + V.light_map_offset;
    // map cells: 8 bytes each {block, item + 1, lit, five mob classes = 0}  (:9241-9269);
    // the loads of all four rounds are issued before the first store
    uint32_t l[4], b[4], it[4];
    bool in[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int cell = lane + 32 * r;
        const int wr = top + cell / kCols, wc = left + cell % kCols;
        in[r] = cell < kCells && wr >= 0 && wr < kMapSize && wc >= 0 && wc < kMapSize;
        const int o = in[r] ? wr * kMapSize + wc : 0;
        l[r] = in[r] ? lit[o] : 0u;
        b[r] = in[r] ? map[o] : 0u;
        it[r] = in[r] ? item[o] : 0u;
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int cell = lane + 32 * r;
        if (cell < kCells) {
            const uint32_t w0 = l[r] > (uint32_t)kLit ? (b[r] | ((it[r] + 1u) & 0xFFu) << 8 | 1u << 16) : 0u;
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

__global__ void __launch_bounds__(kBlockThreads) k_record_rows(const __grid_constant__ Params P) {
    __shared__ Shared S;   // 9 KB
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (warp == 0) {
        const int e = blockIdx.x * kBlockEnvs + t;
        if (e < P.n && (P.skip == nullptr || P.skip[e] == 0)) gather_env(P.v, e, t, S);
        else S.env[t] = -1;
    }
    __syncthreads();
    for (int k = warp; k < kBlockEnvs; k += kBlockThreads / 32) write_env(P, S, k, lane);
}

// the envs named by a device-side list (first int32 of every entry), 32 entries per block pass
__global__ void __launch_bounds__(kBlockThreads) k_record_rows_list(const __grid_constant__ Params P) {
    __shared__ Shared S;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int count = *P.count_dev;
    for (int base = blockIdx.x * kBlockEnvs; base < count; base += (int)gridDim.x * kBlockEnvs) {
        if (warp == 0) {
            int e = -1;
            if (base + t < count) e = *reinterpret_cast<const int32_t*>(P.list + (size_t)(base + t) * P.list_stride);
            if (e >= 0 && e < P.v.num_envs) gather_env(P.v, e, t, S);
            else S.env[t] = -1;
        }
        __syncthreads();
        for (int k = warp; k < kBlockEnvs; k += kBlockThreads / 32) write_env(P, S, k, lane);
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
