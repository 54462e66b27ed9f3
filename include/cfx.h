/*
 * cfx.h -- C ABI of the B200 policy-rollout forward for craftax.cu.
 *
 * The reference keeps its whole host side `static` in one translation unit
 * (craftax_full.cu) and is reused by #include under -DCRAFTAX_CU_LIB; it has
 * no exported ABI.  Each entry point below therefore cites the reference
 * function whose job it takes over inside the `run` rollout loop
 * (cu_rollout_step, craftax_full.cu:12022-12087).
 *
 * Conventions: plain pointers and sizes only; `stream` arguments are
 * cudaStream_t passed as void* (NULL = the handle's own non-blocking stream);
 * every function returns a cfx_status and never exits the process (the
 * reference prints and exit(1)s, craftax_full.cu:8635-8642); cfx_last_error()
 * gives the message for the calling thread.  All device pointers must belong
 * to the handle's device.  There is no CPU fallback: without a usable GPU and
 * the compiled kernels every compute call fails.
 */
#ifndef CFX_H
#define CFX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CFX_OBS_FEATURES 843 /* CF_NN_OBS,     craftax_full.cu:9089  */
#define CFX_OBS_MAP 792      /* CF_NN_MAP,     craftax_full.cu:9091  */
#define CFX_OBS_TAIL 51      /* CF_NN_TAIL,    craftax_full.cu:9092  */
#define CFX_RECORD_BYTES 996 /* CF_TRAIN_OBS,  craftax_full.cu:9111  */
/* classic game: record and feature count (OBS_DIM_COMPACT, OBS_DIM; craftax_classic.cu:59, :40) */
#define CFX_CLASSIC_RECORD_BYTES 148
#define CFX_CLASSIC_OBS_FEATURES 1345
#define CFX_GAME_FULL 0
#define CFX_GAME_CLASSIC 1

typedef enum cfx_status {
    CFX_OK = 0,
    CFX_ERR_INVALID = 1,        /* bad argument (null, size, alignment, n % 32) */
    CFX_ERR_CUDA = 2,           /* a CUDA runtime/driver call failed            */
    CFX_ERR_DEVICE_TIMEOUT = 3, /* a bounded wait inside a kernel gave up       */
    CFX_ERR_IO = 4,             /* checkpoint file problem                      */
    CFX_ERR_UNSUPPORTED = 5     /* shape/precision not built into this library  */
} cfx_status;

/* GEMM operand type of the forward.  Accumulation, the MinGRU cell, the
 * recurrent state and every output are fp32 in all modes. */
typedef enum cfx_precision {
    CFX_PREC_FP32 = 0, /* CUDA-core fmaf in the scalar reference's summation order
                          (role of CRAFTAX_VERIFY_FP32, craftax_full.cu:12513)   */
    CFX_PREC_F16 = 1,  /* fused tcgen05 kernel, fp16 operands (11-bit significand,
                          the same as tf32, at the bf16 rate)                    */
    CFX_PREC_BF16 = 2, /* fused tcgen05 kernel, bf16 operands (the reference's
                          CF_GEMM_BF16 mode, craftax_full.cu:11309).  A throughput
                          point only: its 8-bit significand misses the accuracy
                          gates the fp16 mode meets (greedy-action agreement with
                          the fp32 path about 99.2 % against 99.5 % required)    */
    CFX_PREC_TF32 = 3  /* reserved (the reference's cublasSgemm TF32 mode,
                          craftax_full.cu:11297): not built, create and
                          set_precision return CFX_ERR_UNSUPPORTED; fp16 operands
                          carry the same 11-bit significand                      */
} cfx_precision;

typedef struct cfx_policy cfx_policy;

/* Number of fp32 parameters of the flat arena
 * W_enc[843][H] | b_enc[H] | W_gru[L][3H][H] | W_a[A][H] | b_a[A] | W_v[H] | b_v
 * (CF_NN_PARAM_COUNT, craftax_full.cu:9094-9102). */
size_t cfx_param_count(int hidden, int layers, int num_actions);

/* Replaces cu_policy_init (craftax_full.cu:11819-11907): allocates the
 * parameter arena, operand mirrors, the zeroed recurrent state [L][n][H], the
 * device step counter (= 0) and a non-blocking stream on `device`.
 * num_envs must be a positive multiple of 32 (craftax_full.cu:11820).
 * Shapes: CFX_PREC_FP32 takes any hidden size that is a multiple of 32 up to
 * 512; the fused kernel (CFX_PREC_F16 / CFX_PREC_BF16) is built for hidden 256
 * and 128, 1..4 layers and 43 actions, anything else returns
 * CFX_ERR_UNSUPPORTED.
 * Weights start as zeros; call one of the three setters below. */
int cfx_policy_create(cfx_policy** out, int device, int num_envs, int hidden,
                      int layers, int num_actions, int precision);

/* Replaces cu_policy_free (craftax_full.cu:11909-11921). */
int cfx_policy_destroy(cfx_policy* p);

/* Copies a full arena (host pointer, or device pointer when on_device != 0)
 * and rebuilds the operand mirrors -- the job of cu_params_refresh_bf16 +
 * cu_pack_wav (craftax_full.cu:11805-11817), also what a trainer calls after
 * each optimiser step (craftax_full.cu:13343-13344). */
int cfx_policy_set_weights(cfx_policy* p, const float* arena, size_t count, int on_device);

/* Copies the fp32 arena back to host memory. */
int cfx_policy_get_weights(cfx_policy* p, float* host_arena, size_t count);

/* The reference's own initialiser: seven segments drawn U(+-1/sqrt(fan_in))
 * from Philox4_32_10(seed, subsequence = segment, offset = index)
 * (k_nn_init_weights craftax_full.cu:9123-9131, segments :11832-11845;
 * the reference passes seed 1234). */
int cfx_policy_init_weights(cfx_policy* p, uint64_t seed);

/* CFW1 checkpoint: 16-byte header {0x31574643, hidden, layers, param_count}
 * then the fp32 arena (cu_save_weights / cu_load_weights,
 * craftax_full.cu:12244-12293).  Load validates all four header words. */
int cfx_policy_save_cfw1(cfx_policy* p, const char* path);
int cfx_policy_load_cfw1(cfx_policy* p, const char* path);

/* Switches the operand type (the reference's CF_GEMM_BF16 / math-mode
 * switches, craftax_full.cu:11306-11312, 12512-12514) and rebuilds mirrors. */
int cfx_policy_set_precision(cfx_policy* p, int precision);
int cfx_policy_get_precision(const cfx_policy* p);

/* Device pointer to the live recurrent state, fp32 [layers][num_envs][hidden]
 * (CuPolicy.h_state, craftax_full.cu:11761, element l*H*n + e*H + k as indexed
 * by k_mingru_epi_fwd :9361), and a zero fill of it. */
float* cfx_policy_state(cfx_policy* p);
int cfx_policy_reset_state(cfx_policy* p, void* stream);

/* Device step counter = Philox sampler offset (CuPolicy.step_ctr,
 * craftax_full.cu:11773; k_bump_ctr :9770).  Reading it on the device keeps
 * the forward replayable from a CUDA graph. */
int cfx_policy_set_step(cfx_policy* p, uint64_t step, void* stream);
int cfx_policy_get_step(cfx_policy* p, uint64_t* step);
int cfx_policy_bump_step(cfx_policy* p, void* stream);

/* The handle's stream; number of kernels the last forward launched. */
void* cfx_policy_stream(cfx_policy* p);
int cfx_policy_last_launches(const cfx_policy* p);

/* One batched policy forward: everything cu_rollout_step does between "the
 * record row is complete" and "the env action slots are filled"
 * (k_expand_obs :10028, encoder GEMM + k_add_bias :11954-11962, cu_gru_chain
 * :11978, head GEMM :12040-12045, k_value_sample :9714).
 *
 * Inputs (device): records uint8 [n][996] (16-byte aligned base);
 * prev_terminals float [n] (CuVec.d_terminals; non-zero zeroes that env's
 * state before use; NULL = none); uniforms float [n] or NULL.  With NULL the
 * kernel draws u = curand_uniform(Philox4_32_10(seed ^ 0xA5A5A5A5A5A5A5A5,
 * subsequence = env_offset + e, offset = device step counter)) exactly as
 * k_value_sample does (:9733-9736).
 * Outputs (device, any may be NULL except actions): env_actions float [n]
 * (CuVec.d_actions, read back by the env step), actions int32 [n], logprobs
 * float [n], values float [n]; logits_av float [n][A+1] = logits and value
 * WITH biases added (the reference's scratch holds them before the bias add,
 * :9725-9730), 16-byte aligned base; r_state [L][n][H] = post-zero state inputs for BPTT
 * (:9370-9375), 16-byte aligned; fp32, or bf16 (__float2bfloat16 of the same
 * values, the reference's r_state_bf16 mode) when r_state_bf16 != 0.
 * The recurrent state is updated in place.  The step counter is bumped on
 * the device after the forward when bump_step != 0.
 * No allocation, no host synchronisation and no host-varying kernel argument
 * happens inside: the call is capturable in a CUDA graph. */
typedef struct cfx_forward_io {
    const uint8_t* records;
    const float* prev_terminals;
    const float* uniforms;
    float* env_actions;
    int32_t* actions;
    float* logprobs;
    float* values;
    float* logits_av;
    float* r_state;
    uint64_t seed;
    uint64_t env_offset;
    int bump_step;
    int r_state_bf16; /* 1: r_state points to bf16 [L][n][H] instead of fp32 */
} cfx_forward_io;

int cfx_policy_forward(cfx_policy* p, const cfx_forward_io* io, void* stream);

/* Synchronises `stream` (NULL = the handle's stream) and reports a device-side failure of
 * any forward since the last check: every wait inside the fused kernel is bounded, and a
 * wait that gives up ends the kernel and leaves a status word behind
 * (CFX_ERR_DEVICE_TIMEOUT).  The reference has no counterpart (its kernels cannot time
 * out; errors surface through CU_CHECK, craftax_full.cu:8635). */
int cfx_policy_check(cfx_policy* p, void* stream);

/* Self-test of the device-side timeout path (no reference counterpart): one thread block
 * waits, with a limit of `limit_ms` milliseconds, on a barrier nothing arrives on, gives up and
 * reports through the status word.  Returns CFX_ERR_DEVICE_TIMEOUT when the mechanism works
 * (the expected result), another error otherwise.  The kernel ends normally; the CUDA context
 * stays usable. */
int cfx_selftest_wait_timeout(int device, unsigned limit_ms);

/* Same forward with HOST buffers (pinned for full copy speed): copies
 * records/prev_terminals/uniforms to handle-owned device staging, runs
 * cfx_policy_forward, copies every non-NULL output back and synchronises.
 * With the fused kernel and at least 65,536 envs the records go up in slices
 * of >= 32,768 envs on a second stream and the kernel is launched once per
 * slice behind them (same results; cfx_policy_last_launches counts them). */
int cfx_policy_forward_host(cfx_policy* p, const cfx_forward_io* host_io);

/* Strict-fp32 forward for callers that cannot allocate device memory while they run -- a
 * rollout worker living inside another runtime that owns the device heap, or a loop that
 * cannot afford cudaMalloc's device-wide synchronisation or its failure on a fragmented heap.
 * It has no counterpart in the reference (which allocates all scratch in cu_policy_init).
 * The caller passes everything persistent itself (all device pointers): the fp32 arena
 * `params`, the recurrent state [layers][num_envs][hidden] (updated in place), the inputs and
 * outputs in `io` (as for cfx_policy_forward; bump_step is ignored), and `step_ctr`, the
 * device counter holding the Philox offset (NULL = 0).  Scratch (transposed gate matrices,
 * two layer buffers, logits) lives in one fixed 5.5 MB device array inside the library,
 * resident on every GPU that loads it: hidden must be 256, layers <= 4, num_actions <= 63,
 * num_envs <= 1024 and a multiple of 32; larger sizes are rejected with CFX_ERR_INVALID.
 * io->records must be 16-byte aligned, as for cfx_policy_forward.
 * The first call on a device looks the array's address up (cudaGetSymbolAddress) and must
 * therefore come before any stream capture (a first call on a capturing stream is rejected).
 * The address is kept for the life of the process: after cudaDeviceReset the library has to be
 * reloaded.  No call allocates or frees.  All calls share the array: calls that overlap on
 * the GPU race on it.  Results equal cfx_policy_forward with CFX_PREC_FP32 bit for bit (the
 * same kernels in the same order). */
int cfx_strict_forward_static(int device, const float* params, int hidden, int layers,
                              int num_actions, int num_envs, float* state,
                              const cfx_forward_io* io, const uint64_t* step_ctr, void* stream);

/* Stand-alone stages, for the reference's bitwise gates.
 * cfx_expand_obs: records -> fp32 features [n][843], bit-exact image of
 * k_expand_obs (:10028-10053).  cfx_sample_actions: logits [n][ld] (biases
 * included) + uniforms -> action, logprob; the arithmetic of
 * cf_nn_sample_action (:9147-9165).  cfx_philox_uniforms: the uniforms the
 * forward would draw for (seed, env_offset, step). */
int cfx_expand_obs(int device, const uint8_t* records, float* features, int n, void* stream);
int cfx_sample_actions(int device, const float* logits, int ld, int num_actions,
                       const float* uniforms, int n, int32_t* actions, float* logprobs,
                       void* stream);
int cfx_philox_uniforms(int device, uint64_t seed, uint64_t env_offset, uint64_t step,
                        int n, float* uniforms, void* stream);

/* Thin device-memory and timing helpers so that C, C++ or ctypes callers need
 * no other CUDA binding (cudaMalloc / cudaMemcpyAsync / cudaEvent wrappers). */
int cfx_device_count(int* count);
int cfx_device_name(int device, char* buf, size_t len, int* sm_count, int* cc_major, int* cc_minor);
int cfx_device_alloc(int device, void** ptr, size_t bytes);
int cfx_device_free(int device, void* ptr);
int cfx_host_alloc_pinned(void** ptr, size_t bytes);
int cfx_host_free_pinned(void* ptr);
int cfx_memcpy_h2d(int device, void* dst, const void* src, size_t bytes, void* stream);
int cfx_memcpy_d2h(int device, void* dst, const void* src, size_t bytes, void* stream);
int cfx_memset(int device, void* dst, int value, size_t bytes, void* stream);
int cfx_stream_sync(int device, void* stream);
int cfx_timer_create(int device, void** timer);
int cfx_timer_destroy(void* timer);
int cfx_timer_start(void* timer, void* stream); /* cudaEventRecord on `stream` */
int cfx_timer_stop(void* timer, void* stream);
int cfx_timer_elapsed_ms(void* timer, float* ms); /* synchronises on the stop event */

const char* cfx_last_error(void);
const char* cfx_version(void);

/* ---- record write (reference k_record_obs / cf_record_env_warp, craftax_full.cu:9180-9297,
 * call site cu_encode_step :11933-11953) ------------------------------------------------
 * Writes the 996-byte compact record of every env from the env state the reference keeps on
 * the device, byte for byte what k_record_obs writes: 99 view cells (9 rows x 11 columns
 * around the player) x 8 bytes {block, item + 1, lit flag, five mob-class bytes (type + 1)},
 * zero for cells that are off the map or not lit (light_map <= 12), then the 51 raw fp32
 * scalars of craftax_encode_scalar_observation_tail_at (:2429-2487).
 * cfx_env_view describes that state without naming the reference's structs: the SoA fields
 * (CF_SOA_FIELDS, :620-690; element i of env e of a field is field[i * num_envs + e], bool
 * fields are one byte) and the three byte maps [9][48][48] inside the per-env block of
 * state_stride bytes.  All pointers are device pointers; nothing is copied or retained.
 * skip (optional, uint8 [n]): envs whose flag is non-zero are left untouched (the reference
 * records those after their reset has been joined, k_record_obs_list :9303-9319);
 * cfx_record_obs_list writes exactly the envs listed in `list` (entries of list_stride bytes
 * whose first int32 is the env index, e.g. CraftaxResetRec :8707-8711; *count_dev entries).
 * Asynchronous on `stream`, no allocation, capturable in a CUDA graph. */
typedef struct cfx_env_view {
    int32_t num_envs;
    const uint8_t* state_base;
    uint64_t state_stride;
    uint64_t map_offset, item_map_offset, light_map_offset;
    const int32_t* player_position; /* [2]: row, column */
    const int32_t* player_level;
    const int32_t* player_direction;
    const float* player_health;
    const int32_t* player_food;
    const int32_t* player_drink;
    const int32_t* player_energy;
    const int32_t* player_mana;
    const uint8_t* is_sleeping;
    const uint8_t* is_resting;
    const int32_t* player_xp;
    const int32_t* player_dexterity;
    const int32_t* player_strength;
    const int32_t* player_intelligence;
    const int32_t* inv_wood;
    const int32_t* inv_stone;
    const int32_t* inv_coal;
    const int32_t* inv_iron;
    const int32_t* inv_diamond;
    const int32_t* inv_sapling;
    const int32_t* inv_pickaxe;
    const int32_t* inv_sword;
    const int32_t* inv_bow;
    const int32_t* inv_arrows;
    const int32_t* inv_torches;
    const int32_t* inv_ruby;
    const int32_t* inv_sapphire;
    const int32_t* inv_books;
    const int32_t* inv_armour;          /* [4] */
    const int32_t* inv_potions;         /* [6] */
    const uint8_t* learned_spells;      /* [2] */
    const int32_t* sword_enchantment;
    const int32_t* bow_enchantment;
    const int32_t* armour_enchantments; /* [4] */
    const int32_t* boss_timesteps_to_spawn_this_round;
    const float* light_level;
    const int32_t* monsters_killed;     /* [9] */
    const int32_t* mob_position;        /* [5 classes][9 levels][3 slots][2] */
    const uint8_t* mob_mask;            /* [5][9][3] */
    const int32_t* mob_type_id;         /* [5][9][3] */
} cfx_env_view;

int cfx_record_obs(int device, const cfx_env_view* view, uint8_t* records, int n,
                   const uint8_t* skip, void* stream);
int cfx_record_obs_list(int device, const cfx_env_view* view, uint8_t* records, const void* list,
                        int list_stride, const int* count_dev, void* stream);

/* ---- classic game (reference craftax_classic.cu, boundary Rollout::step in
 * main_classic.cu:439-474) ------------------------------------------------------------
 * Same handle type and the same calls as the full game (set_weights, state, step counter,
 * forward, forward_host); what differs is the record (148 bytes: 63 block ids, 63 mob bit
 * masks, 12 inventory counts, health/food/drink/energy, direction, sleeping flag, light as
 * raw fp32; craftax_classic.cu:50-59), the encoder (a gather of W_enc rows in the order of
 * encode_obs_kernel, :1714-1751) and the arena, whose W_enc has 1345 rows (:1526-1533).
 * CFX_PREC_FP32 follows the reference's summation order; CFX_PREC_F16 / CFX_PREC_BF16 run the
 * fused tcgen05 kernel (hidden 256, 17 actions), whose expand turns the record into one-hot
 * operand rows in tensor memory and whose encoder is a dense MMA over the 1345 features.
 * cfx_forward_io.records then holds uint8 [n][148]; prev_terminals holds float flags
 * (cfx_classic_done_to_terminals converts the rollout's int8 r_done row). */
size_t cfx_classic_param_count(int hidden, int layers, int num_actions);
int cfx_policy_create_classic(cfx_policy** out, int device, int num_envs, int hidden,
                              int layers, int num_actions, int precision);
/* Replaces expand_obs_kernel (craftax_classic.cu:1265-1301): uint8 [n][148] -> fp32 [n][1345]
 * (device pointers). */
int cfx_classic_expand_obs(int device, const uint8_t* records, float* out, int num_envs,
                           void* stream);
/* int8 done flags -> float terminal flags (device pointers). */
int cfx_classic_done_to_terminals(int device, const int8_t* done, float* out, int num_envs,
                                  void* stream);

/* Classic game: the 148-byte record of every env from the reference's classic device state, byte
 * for byte what record_obs_kernel / write_compact_obs write (craftax_classic.cu:1574-1604,
 * :1884-1890; view gathering :1061-1126): 63 block ids of the 7 x 9 view around the player (1 =
 * out of bounds), 63 mob bit masks (1 zombie, 2 cow, 4 skeleton, 8 arrow), 12 inventory counts,
 * health, food, drink, energy, direction, sleeping flag, light level as raw fp32.  The view names
 * the fields of the reference's EnvSoA (:134-194) it reads: per-env fields are [n], slot-major
 * fields [slots][n]; map_packed holds map_stride bytes per env, 64 rows of 32 bytes, two columns
 * per byte with the even column in the low nibble. */
typedef struct cfx_classic_env_view {
    int32_t num_envs;
    const uint8_t* map_packed;
    uint64_t map_stride;
    const int16_t* player_r;
    const int16_t* player_c;
    const int8_t* player_dir;
    const int8_t* health;
    const int8_t* food;
    const int8_t* drink;
    const int8_t* energy;
    const uint8_t* is_sleeping;
    const int8_t* inv;           /* [12][n] */
    const int16_t* zombie_r;     /* [3][n] */
    const int16_t* zombie_c;
    const uint8_t* zombie_mask;
    const int16_t* cow_r;        /* [3][n] */
    const int16_t* cow_c;
    const uint8_t* cow_mask;
    const int16_t* skel_r;       /* [2][n] */
    const int16_t* skel_c;
    const uint8_t* skel_mask;
    const int16_t* arrow_r;      /* [3][n] */
    const int16_t* arrow_c;
    const uint8_t* arrow_mask;
    const float* light_level;
} cfx_classic_env_view;

int cfx_classic_record_obs(int device, const cfx_classic_env_view* view, uint8_t* records, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CFX_H */
