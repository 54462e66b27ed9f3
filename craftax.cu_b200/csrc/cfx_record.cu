// Record write: env state -> 996-byte compact records (reference k_record_obs /
// cf_record_env_warp, craftax_full.cu:9180-9297; scalar tail :2429-2487).
//
// One warp per env, like the reference, but nothing in it is serial: the 14 mob slots of the
// player's level are examined by 14 lanes at once and broadcast with shuffles (the reference
// builds the list on lane 0), and the 51 tail scalars are produced by 51 lanes from a table of
// (field, element, conversion) entries that the host fills from the caller's view (the
// reference computes them on lane 0 and stores them cooperatively).  The bytes are the same:
// the same predicates, the same "last slot of a class wins a cell" order, the same float
// expressions (sqrtf(x) * 0.1f, x * 0.1f, x * 0.5f, x * 0.25f; no fused multiply-add can form).
// HBM traffic per env: 996 B written, 27 map sectors (9 rows of 11 bytes in three maps) and
// ~60 SoA words read; the SoA words of the eight envs of a block share sectors.
#include <cuda_runtime.h>

#include "cfx_common.cuh"

namespace cfx {
namespace record {

constexpr int kRows = 9, kCols = 11, kCells = kRows * kCols;   // view around the player
constexpr int kMapSize = 48, kLevels = 9, kMobTypes = 8, kClasses = 5, kSlots = 3;
constexpr int kLit = 12;                                       // light_map > 12 = visible
constexpr int kKilledToClear = 8;
constexpr int kWarpsPerBlock = 8;

enum Op : uint8_t { OP_I32_MUL, OP_I32_SQRT10, OP_F32_MUL, OP_BOOL, OP_DIR, OP_KILLED, OP_BOSS };
struct TailSrc {
    const void* field;   // SoA field
    int32_t elem;        // element of the field (OP_DIR: the direction this output stands for)
    Op op;
    float mul;
};
struct Params {
    cfx_env_view v;
    TailSrc tail[kTail];
    uint8_t* records;
    const uint8_t* skip;
    const uint8_t* list;
    int list_stride;
    const int* count_dev;
    int n;
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

__device__ __forceinline__ void record_env(const Params& P, int e, int lane) {
    const cfx_env_view& V = P.v;
    const int n = V.num_envs;
    uint8_t* rec = P.records + (size_t)e * kRec;
    const int level = soa(V.player_level, 0, n, e);
    const int mob_level = jax_index(level, kLevels);
    const int top = soa(V.player_position, 0, n, e) - kRows / 2;
    const int left = soa(V.player_position, 1, n, e) - kCols / 2;
    const uint8_t* blk = V.state_base + (size_t)e * V.state_stride;
    const uint8_t* light = blk + V.light_map_offset;

    // ---- visible mobs of the player's level: lane m examines (class m / 3, slot m % 3);
    // packed = valid | cell << 8 | channel << 4 | value  (:9195-9236)
    uint32_t mine = 0;
    {
        const int c = lane / kSlots, i = lane % kSlots;
        if (c < kClasses && i < (c == 2 ? 2 : 3)) {
            const int idx = mob_index(c, mob_level, i);
            const int type_id = soa(V.mob_type_id, idx, n, e);
            const bool mask = soa(V.mob_mask, idx, n, e) != 0;
            if (type_id >= 0 && type_id < kMobTypes && mask) {
                const int mr = soa(V.mob_position, idx * 2, n, e), mc = soa(V.mob_position, idx * 2 + 1, n, e);
                const int lr = mr - top, lc = mc - left;
                if (lr >= 0 && lr < kRows && lc >= 0 && lc < kCols && mr >= 0 && mr < kMapSize && mc >= 0 &&
                    mc < kMapSize && light[(mob_level * kMapSize + mr) * kMapSize + mc] > kLit)
                    mine = 0x80000000u | (uint32_t)(lr * kCols + lc) << 8 | (uint32_t)(3 + c) << 4 |
                           (uint32_t)(type_id + 1);
            }
        }
    }
    uint32_t mobs[kClasses * kSlots];
#pragma unroll
    for (int m = 0; m < kClasses * kSlots; m++) mobs[m] = __shfl_sync(0xFFFFFFFFu, mine, m);

    // ---- map cells: 8 bytes each {block, item + 1, lit, five mob classes}  (:9241-9269)
    const uint8_t* map = blk + V.map_offset + (size_t)level * kMapSize * kMapSize;
    const uint8_t* item = blk + V.item_map_offset + (size_t)level * kMapSize * kMapSize;
    const uint8_t* lit = light + (size_t)level * kMapSize * kMapSize;
    for (int cell = lane; cell < kCells; cell += 32) {
        const int wr = top + cell / kCols, wc = left + cell % kCols;
        uint64_t w = 0;
        if (wr >= 0 && wr < kMapSize && wc >= 0 && wc < kMapSize && lit[wr * kMapSize + wc] > kLit)
            w = (uint64_t)map[wr * kMapSize + wc] | (uint64_t)(uint8_t)(item[wr * kMapSize + wc] + 1) << 8 |
                1ull << 16;
        // slots in class-major, slot-minor order: a later slot of the same class overwrites
#pragma unroll
        for (int m = 0; m < kClasses * kSlots; m++) {
            const uint32_t pk = mobs[m];
            if ((pk & 0x80000000u) && (int)((pk >> 8) & 0xFFu) == cell) {
                const int sh = 8 * (int)((pk >> 4) & 0xFu);
                w = (w & ~(0xFFull << sh)) | (uint64_t)(pk & 0xFu) << sh;
            }
        }
        uint32_t* dst = reinterpret_cast<uint32_t*>(rec + (size_t)cell * 8);   // 4-byte aligned (996 = 4 x 249)
        dst[0] = (uint32_t)w;
        dst[1] = (uint32_t)(w >> 32);
    }

    // ---- scalar tail: output j from P.tail[j]  (:2429-2487)
    for (int j = lane; j < kTail; j += 32) {
        const TailSrc t = P.tail[j];
        float out;
        switch (t.op) {
        case OP_I32_MUL:
            out = (float)soa((const int32_t*)t.field, t.elem, n, e) * t.mul;
            break;
        case OP_I32_SQRT10:
            out = sqrtf((float)soa((const int32_t*)t.field, t.elem, n, e)) * (1.0f / 10.0f);
            break;
        case OP_F32_MUL:
            out = soa((const float*)t.field, t.elem, n, e);
            if (t.mul != 1.0f) out = out * t.mul;
            break;
        case OP_BOOL:
            out = soa((const uint8_t*)t.field, t.elem, n, e) != 0 ? 1.0f : 0.0f;
            break;
        case OP_DIR:
            out = soa((const int32_t*)t.field, 0, n, e) - 1 == t.elem ? 1.0f : 0.0f;
            break;
        case OP_KILLED:
            out = soa((const int32_t*)t.field, level, n, e) >= kKilledToClear ? 1.0f : 0.0f;
            break;
        default: {   // OP_BOSS: craftax_wg_is_boss_vulnerable (:1988-2003)
            bool any = false;
            for (int i = 0; i < 3; i++) any = any || soa(V.mob_mask, mob_index(0, mob_level, i), n, e) != 0;
            for (int i = 0; i < 2; i++) any = any || soa(V.mob_mask, mob_index(2, mob_level, i), n, e) != 0;
            out = !any && soa(V.boss_timesteps_to_spawn_this_round, 0, n, e) <= 0 ? 1.0f : 0.0f;
        }
        }
        *reinterpret_cast<float*>(rec + kMap + 4 * j) = out;
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) k_record_rows(const __grid_constant__ Params P) {
    const int lane = threadIdx.x & 31;
    const int e = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (e >= P.n) return;
    if (P.skip != nullptr && P.skip[e] != 0) return;
    record_env(P, e, lane);
}

// the envs named by a device-side list (first int32 of every entry), grid-strided
__global__ void __launch_bounds__(kWarpsPerBlock * 32) k_record_rows_list(const __grid_constant__ Params P) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int count = *P.count_dev;
    for (int idx = blockIdx.x * kWarpsPerBlock + warp; idx < count; idx += (int)gridDim.x * kWarpsPerBlock) {
        const int e = *reinterpret_cast<const int32_t*>(P.list + (size_t)idx * P.list_stride);
        if (e >= 0 && e < P.v.num_envs) record_env(P, e, lane);
        __syncwarp();
    }
}

// the 51 outputs in the order of craftax_encode_scalar_observation_tail_at
static int fill_tail(const cfx_env_view& v, TailSrc* t) {
    int k = 0;
    auto add = [&](const void* f, int elem, Op op, float mul) {
        t[k].field = f; t[k].elem = elem; t[k].op = op; t[k].mul = mul;
        k++;
    };
    const int32_t* sq[10] = {v.inv_wood, v.inv_stone, v.inv_coal, v.inv_iron, v.inv_diamond,
                             v.inv_sapphire, v.inv_ruby, v.inv_sapling, v.inv_torches, v.inv_arrows};
    for (int i = 0; i < 10; i++) add(sq[i], 0, OP_I32_SQRT10, 0.1f);
    add(v.inv_books, 0, OP_I32_MUL, 1.0f / 2.0f);
    add(v.inv_pickaxe, 0, OP_I32_MUL, 1.0f / 4.0f);
    add(v.inv_sword, 0, OP_I32_MUL, 1.0f / 4.0f);
    add(v.sword_enchantment, 0, OP_I32_MUL, 1.0f);
    add(v.bow_enchantment, 0, OP_I32_MUL, 1.0f);
    add(v.inv_bow, 0, OP_I32_MUL, 1.0f);
    for (int i = 0; i < 6; i++) add(v.inv_potions, i, OP_I32_SQRT10, 0.1f);
    add(v.player_health, 0, OP_F32_MUL, 1.0f / 10.0f);
    const int32_t* tenth[8] = {v.player_food, v.player_drink, v.player_energy, v.player_mana, v.player_xp,
                               v.player_dexterity, v.player_strength, v.player_intelligence};
    for (int i = 0; i < 8; i++) add(tenth[i], 0, OP_I32_MUL, 1.0f / 10.0f);
    for (int i = 0; i < 4; i++) add(v.player_direction, i, OP_DIR, 0.0f);
    for (int i = 0; i < 4; i++) add(v.inv_armour, i, OP_I32_MUL, 1.0f / 2.0f);
    for (int i = 0; i < 4; i++) add(v.armour_enchantments, i, OP_I32_MUL, 1.0f);
    add(v.light_level, 0, OP_F32_MUL, 1.0f);
    add(v.is_sleeping, 0, OP_BOOL, 0.0f);
    add(v.is_resting, 0, OP_BOOL, 0.0f);
    add(v.learned_spells, 0, OP_BOOL, 0.0f);
    add(v.learned_spells, 1, OP_BOOL, 0.0f);
    add(v.player_level, 0, OP_I32_MUL, 1.0f / 10.0f);
    add(v.monsters_killed, 0, OP_KILLED, 0.0f);
    add(v.mob_mask, 0, OP_BOSS, 0.0f);
    return k;
}

static int make_params(const char* who, const cfx_env_view* view, uint8_t* records, Params* P) {
    CFX_REQUIRE(view != nullptr && records != nullptr, "%s: bad argument", who);
    CFX_REQUIRE(view->num_envs > 0 && view->state_base != nullptr && view->state_stride > 0,
                "%s: the view has no envs or no state block", who);
    CFX_REQUIRE(((uintptr_t)records & 3) == 0, "%s: records must be 4-byte aligned", who);
    P->v = *view;
    const int k = fill_tail(*view, P->tail);
    CFX_REQUIRE(k == kTail, "%s: internal: %d tail outputs", who, k);
    for (int j = 0; j < kTail; j++)
        CFX_REQUIRE(P->tail[j].field != nullptr, "%s: the field behind tail output %d is NULL", who, j);
    CFX_REQUIRE(view->player_position != nullptr && view->mob_position != nullptr && view->mob_type_id != nullptr &&
                    view->boss_timesteps_to_spawn_this_round != nullptr,
                "%s: a position / mob field of the view is NULL", who);
    P->records = records;
    P->skip = nullptr; P->list = nullptr; P->list_stride = 0; P->count_dev = nullptr;
    P->n = view->num_envs;
    return CFX_OK;
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
    const unsigned blocks = (unsigned)(((size_t)n + record::kWarpsPerBlock - 1) / record::kWarpsPerBlock);
    record::k_record_rows<<<blocks, record::kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(P);
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
    // as many warps as the reference uses for its list pass (at most 128 blocks of 8, :11941)
    int blocks = (view->num_envs + record::kWarpsPerBlock - 1) / record::kWarpsPerBlock;
    if (blocks > 128) blocks = 128;
    record::k_record_rows_list<<<blocks, record::kWarpsPerBlock * 32, 0, (cudaStream_t)stream>>>(P);
    CFX_CUDA(cudaGetLastError());
    return CFX_OK;
}
