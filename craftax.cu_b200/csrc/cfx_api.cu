// C-ABI layer: the policy handle and every extern "C" entry point of cfx.h.
#include <cstdarg>
#include <cstdlib>
#include <cmath>
#include <new>

#include "cfx_common.cuh"
#include "cfx_fused.h"
#include "cfx_strict.h"

namespace cfx {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
    return CFX_ERR_CUDA;
}

}  // namespace cfx

using namespace cfx;

constexpr int kHostSlicesMax = 8;
constexpr size_t kHostSliceEnvs = 32768;   // smallest slice of the pipelined host-buffer forward

// The handle: role of CuPolicy (craftax_full.cu:11758-11796).
struct cfx_policy {
    int device = 0;
    int n = 0, H = 0, L = 0, A = 0;
    int game = CFX_GAME_FULL, obs = kObs, rec_bytes = kRec;
    int precision = CFX_PREC_FP32;
    size_t param_count = 0;
    float* params = nullptr;        // fp32 arena (device)
    float* gates_t = nullptr;       // strict path: transposed gate matrices
    float* state = nullptr;         // [L][n][H]
    float* scratch_h[2] = {nullptr, nullptr};  // strict path layer ping-pong
    float* logits_scratch = nullptr;           // [n][A+1] when the caller passes none
    unsigned long long* step_ctr = nullptr;
    cudaStream_t stream = nullptr;
    FusedPlan* fused = nullptr;
    int last_launches = 0;
    // device staging of cfx_policy_forward_host
    uint8_t* st_records = nullptr;
    float* st_terminals = nullptr;
    float* st_uniforms = nullptr;
    float* st_env_actions = nullptr;
    int32_t* st_actions = nullptr;
    float* st_logprobs = nullptr;
    float* st_values = nullptr;
    float* st_logits = nullptr;
    float* st_r_state = nullptr;
    // cfx_policy_forward_host: copy stream and per-slice events of the pipelined upload
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t slice_ready[kHostSlicesMax] = {};
    cudaEvent_t host_fence = nullptr;
};

static void free_dev(void* p) {
    if (p) cudaFree(p);
}

static int policy_refresh_mirrors(cfx_policy* p, cudaStream_t st) {
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A, p->obs);
    int rc = launch_transpose_gates(p->params + o.w_gru, p->gates_t, p->H, p->L, st);
    if (rc) return rc;
    if (p->fused) {
        rc = fused_refresh(p->fused, p->params, st);
        if (rc) return rc;
    }
    return CFX_OK;
}

static int policy_ensure_fused(cfx_policy* p) {
    if (p->precision == CFX_PREC_FP32) return CFX_OK;
    if (!fused_supported(p->H, p->L, p->A, p->precision, p->game)) {
        set_error("precision %d is not built for hidden=%d layers=%d actions=%d", p->precision,
                  p->H, p->L, p->A);
        return CFX_ERR_UNSUPPORTED;
    }
    if (p->fused) {
        fused_destroy(p->fused);
        p->fused = nullptr;
    }
    return fused_create(&p->fused, p->device, p->n, p->H, p->L, p->A, p->precision, p->state, p->game);
}

extern "C" {

const char* cfx_last_error(void) { return g_err; }
const char* cfx_version(void) { return "cfx-b200 0.1 (sm_100a)"; }

size_t cfx_param_count(int hidden, int layers, int num_actions) {
    if (hidden <= 0 || layers <= 0 || num_actions <= 0) return 0;
    return ArenaLayout::make(hidden, layers, num_actions).count;
}

static int policy_create(cfx_policy** out, int device, int num_envs, int hidden, int layers,
                         int num_actions, int precision, int game);

int cfx_policy_create(cfx_policy** out, int device, int num_envs, int hidden, int layers,
                      int num_actions, int precision) {
    return policy_create(out, device, num_envs, hidden, layers, num_actions, precision, CFX_GAME_FULL);
}

int cfx_policy_create_classic(cfx_policy** out, int device, int num_envs, int hidden, int layers,
                              int num_actions, int precision) {
    return policy_create(out, device, num_envs, hidden, layers, num_actions, precision, CFX_GAME_CLASSIC);
}

size_t cfx_classic_param_count(int hidden, int layers, int num_actions) {
    if (hidden <= 0 || layers <= 0 || num_actions <= 0) return 0;
    return ArenaLayout::make(hidden, layers, num_actions, kClassicObs).count;
}

int cfx_classic_expand_obs(int device, const uint8_t* records, float* out, int num_envs, void* stream) {
    CFX_REQUIRE(records && out && num_envs > 0, "cfx_classic_expand_obs: bad arguments");
    CFX_GUARD(device);
    return launch_classic_expand(records, out, num_envs, (cudaStream_t)stream);
}

int cfx_classic_done_to_terminals(int device, const int8_t* done, float* out, int num_envs, void* stream) {
    CFX_REQUIRE(done && out && num_envs > 0, "cfx_classic_done_to_terminals: bad arguments");
    CFX_GUARD(device);
    return launch_done_to_terminals(done, out, num_envs, (cudaStream_t)stream);
}

static int policy_create(cfx_policy** out, int device, int num_envs, int hidden, int layers,
                         int num_actions, int precision, int game) {
    CFX_REQUIRE(out != nullptr, "cfx_policy_create: out is NULL");
    *out = nullptr;
    CFX_REQUIRE(num_envs > 0 && num_envs % 32 == 0,
                "cfx_policy_create: num_envs=%d must be a positive multiple of 32", num_envs);
    CFX_REQUIRE(hidden >= 32 && hidden <= 512 && hidden % 32 == 0,
                "cfx_policy_create: hidden=%d must be a multiple of 32 in [32,512]", hidden);
    CFX_REQUIRE(layers >= 1 && layers <= 8, "cfx_policy_create: layers=%d out of [1,8]", layers);
    CFX_REQUIRE(num_actions >= 2 && num_actions <= kMaxActions,
                "cfx_policy_create: num_actions=%d out of [2,%d]", num_actions, kMaxActions);
    CFX_REQUIRE(precision >= CFX_PREC_FP32 && precision <= CFX_PREC_TF32,
                "cfx_policy_create: unknown precision %d", precision);
    int ndev = 0;
    CFX_CUDA(cudaGetDeviceCount(&ndev));
    CFX_REQUIRE(device >= 0 && device < ndev, "cfx_policy_create: device %d of %d", device, ndev);
    CFX_GUARD(device);
    cfx_policy* p = new (std::nothrow) cfx_policy();
    CFX_REQUIRE(p != nullptr, "cfx_policy_create: out of host memory");
    p->device = device;
    p->n = num_envs;
    p->H = hidden;
    p->L = layers;
    p->A = num_actions;
    p->precision = precision;
    p->game = game;
    p->obs = game == CFX_GAME_CLASSIC ? kClassicObs : kObs;
    p->rec_bytes = game == CFX_GAME_CLASSIC ? kClassicRec : kRec;
    p->param_count = ArenaLayout::make(hidden, layers, num_actions, p->obs).count;
    const size_t hn = (size_t)hidden * num_envs;
    int rc = CFX_OK;
    auto fail = [&](int code) {
        cfx_policy_destroy(p);
        return code;
    };
#define CFX_TRY_ALLOC(ptr, bytes)                                                    \
    do {                                                                             \
        cudaError_t _e = cudaMalloc((void**)&(ptr), (bytes));                        \
        if (_e != cudaSuccess) return fail(cuda_fail(_e, "cudaMalloc " #ptr, __FILE__, __LINE__)); \
    } while (0)
    CFX_TRY_ALLOC(p->params, p->param_count * sizeof(float));
    CFX_TRY_ALLOC(p->gates_t, (size_t)layers * 3 * hidden * hidden * sizeof(float));
    CFX_TRY_ALLOC(p->state, (size_t)layers * hn * sizeof(float));
    CFX_TRY_ALLOC(p->scratch_h[0], hn * sizeof(float));
    CFX_TRY_ALLOC(p->scratch_h[1], hn * sizeof(float));
    CFX_TRY_ALLOC(p->logits_scratch, (size_t)num_envs * (num_actions + 1) * sizeof(float));
    CFX_TRY_ALLOC(p->step_ctr, sizeof(unsigned long long));
#undef CFX_TRY_ALLOC
    cudaError_t e = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaStreamCreateWithFlags", __FILE__, __LINE__));
    e = cudaMemsetAsync(p->params, 0, p->param_count * sizeof(float), p->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->state, 0, (size_t)layers * hn * sizeof(float), p->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->step_ctr, 0, sizeof(unsigned long long), p->stream);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemsetAsync", __FILE__, __LINE__));
    rc = policy_ensure_fused(p);
    if (rc) return fail(rc);
    rc = policy_refresh_mirrors(p, p->stream);
    if (rc) return fail(rc);
    e = cudaStreamSynchronize(p->stream);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaStreamSynchronize", __FILE__, __LINE__));
    *out = p;
    return CFX_OK;
}

int cfx_policy_destroy(cfx_policy* p) {
    if (!p) return CFX_OK;
    DeviceGuard g(p->device);   // best effort: the handle is released whatever happens
    if (p->stream) cudaStreamSynchronize(p->stream);
    if (p->fused) fused_destroy(p->fused);
    free_dev(p->params);
    free_dev(p->gates_t);
    free_dev(p->state);
    free_dev(p->scratch_h[0]);
    free_dev(p->scratch_h[1]);
    free_dev(p->logits_scratch);
    free_dev(p->step_ctr);
    free_dev(p->st_records);
    free_dev(p->st_terminals);
    free_dev(p->st_uniforms);
    free_dev(p->st_env_actions);
    free_dev(p->st_actions);
    free_dev(p->st_logprobs);
    free_dev(p->st_values);
    free_dev(p->st_logits);
    free_dev(p->st_r_state);
    for (int i = 0; i < kHostSlicesMax; i++)
        if (p->slice_ready[i]) cudaEventDestroy(p->slice_ready[i]);
    if (p->host_fence) cudaEventDestroy(p->host_fence);
    if (p->copy_stream) cudaStreamDestroy(p->copy_stream);
    if (p->stream) cudaStreamDestroy(p->stream);
    delete p;
    return CFX_OK;
}

int cfx_policy_set_weights(cfx_policy* p, const float* arena, size_t count, int on_device) {
    CFX_REQUIRE(p && arena, "cfx_policy_set_weights: NULL argument");
    CFX_REQUIRE(count == p->param_count, "cfx_policy_set_weights: count %zu != %zu", count,
                p->param_count);
    CFX_GUARD(p->device);
    CFX_CUDA(cudaMemcpyAsync(p->params, arena, count * sizeof(float),
                             on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                             p->stream));
    int rc = policy_refresh_mirrors(p, p->stream);
    if (rc) return rc;
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    return CFX_OK;
}

int cfx_policy_get_weights(cfx_policy* p, float* host_arena, size_t count) {
    CFX_REQUIRE(p && host_arena, "cfx_policy_get_weights: NULL argument");
    CFX_REQUIRE(count == p->param_count, "cfx_policy_get_weights: count %zu != %zu", count,
                p->param_count);
    CFX_GUARD(p->device);
    CFX_CUDA(cudaMemcpyAsync(host_arena, p->params, count * sizeof(float), cudaMemcpyDeviceToHost,
                             p->stream));
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    return CFX_OK;
}

int cfx_policy_init_weights(cfx_policy* p, uint64_t seed) {
    CFX_REQUIRE(p, "cfx_policy_init_weights: NULL handle");
    CFX_GUARD(p->device);
    const ArenaLayout o = ArenaLayout::make(p->H, p->L, p->A, p->obs);
    const float be = 1.0f / sqrtf((float)p->obs), bh = 1.0f / sqrtf((float)p->H);
    const struct { size_t off; size_t count; float bound; } segs[7] = {
        {o.w_enc, (size_t)p->obs * p->H, be}, {o.b_enc, (size_t)p->H, be},
        {o.w_gru, (size_t)p->L * 3 * p->H * p->H, bh}, {o.w_a, (size_t)p->A * p->H, bh},
        {o.b_a, (size_t)p->A, bh}, {o.w_v, (size_t)p->H, bh}, {o.b_v, 1, bh}};
    for (int s = 0; s < 7; s++) {
        int rc = launch_init_uniform(p->params + segs[s].off, (int)segs[s].count, segs[s].bound,
                                     seed, s, p->stream);
        if (rc) return rc;
    }
    int rc = policy_refresh_mirrors(p, p->stream);
    if (rc) return rc;
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    return CFX_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ checkpoint
static const uint32_t kCkptMagic = 0x31574643u;  // "CFW1", craftax_full.cu:12243

extern "C" {

int cfx_policy_save_cfw1(cfx_policy* p, const char* path) {
    CFX_REQUIRE(p && path, "cfx_policy_save_cfw1: NULL argument");
    float* h = (float*)malloc(p->param_count * sizeof(float));
    CFX_REQUIRE(h != nullptr, "cfx_policy_save_cfw1: out of host memory");
    int rc = cfx_policy_get_weights(p, h, p->param_count);
    if (rc) { free(h); return rc; }
    FILE* f = fopen(path, "wb");
    if (!f) {
        free(h);
        set_error("cfx_policy_save_cfw1: cannot write %s", path);
        return CFX_ERR_IO;
    }
    const uint32_t hdr[4] = {kCkptMagic, (uint32_t)p->H, (uint32_t)p->L, (uint32_t)p->param_count};
    bool ok = fwrite(hdr, sizeof(hdr), 1, f) == 1 &&
              fwrite(h, sizeof(float), p->param_count, f) == p->param_count;
    ok = (fclose(f) == 0) && ok;
    free(h);
    if (!ok) {
        set_error("cfx_policy_save_cfw1: short write to %s", path);
        return CFX_ERR_IO;
    }
    return CFX_OK;
}

int cfx_policy_load_cfw1(cfx_policy* p, const char* path) {
    CFX_REQUIRE(p && path, "cfx_policy_load_cfw1: NULL argument");
    FILE* f = fopen(path, "rb");
    if (!f) {
        set_error("cfx_policy_load_cfw1: cannot read %s", path);
        return CFX_ERR_IO;
    }
    uint32_t hdr[4];
    if (fread(hdr, sizeof(hdr), 1, f) != 1 || hdr[0] != kCkptMagic || hdr[1] != (uint32_t)p->H ||
        hdr[2] != (uint32_t)p->L || hdr[3] != (uint32_t)p->param_count) {
        fclose(f);
        set_error("cfx_policy_load_cfw1: %s: bad header (want h%dx%d, %zu params)", path, p->H,
                  p->L, p->param_count);
        return CFX_ERR_IO;
    }
    float* h = (float*)malloc(p->param_count * sizeof(float));
    if (!h) {
        fclose(f);
        set_error("cfx_policy_load_cfw1: out of host memory");
        return CFX_ERR_INVALID;
    }
    size_t got = fread(h, sizeof(float), p->param_count, f);
    fclose(f);
    if (got != p->param_count) {
        free(h);
        set_error("cfx_policy_load_cfw1: %s: truncated", path);
        return CFX_ERR_IO;
    }
    int rc = cfx_policy_set_weights(p, h, p->param_count, 0);
    free(h);
    return rc;
}

int cfx_policy_set_precision(cfx_policy* p, int precision) {
    CFX_REQUIRE(p, "cfx_policy_set_precision: NULL handle");
    CFX_REQUIRE(precision >= CFX_PREC_FP32 && precision <= CFX_PREC_TF32,
                "cfx_policy_set_precision: unknown precision %d", precision);
    if (precision == p->precision) return CFX_OK;
    CFX_GUARD(p->device);
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    const int old = p->precision;
    p->precision = precision;
    if (precision == CFX_PREC_FP32) {
        if (p->fused) {
            fused_destroy(p->fused);
            p->fused = nullptr;
        }
        return CFX_OK;
    }
    int rc = policy_ensure_fused(p);
    if (rc) {
        p->precision = old;
        if (old != CFX_PREC_FP32) policy_ensure_fused(p);
        if (p->fused) fused_refresh(p->fused, p->params, p->stream);
        return rc;
    }
    rc = fused_refresh(p->fused, p->params, p->stream);
    if (rc) return rc;
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    return CFX_OK;
}

int cfx_policy_get_precision(const cfx_policy* p) { return p ? p->precision : -1; }

float* cfx_policy_state(cfx_policy* p) { return p ? p->state : nullptr; }

int cfx_policy_reset_state(cfx_policy* p, void* stream) {
    CFX_REQUIRE(p, "cfx_policy_reset_state: NULL handle");
    CFX_GUARD(p->device);
    cudaStream_t st = stream ? (cudaStream_t)stream : p->stream;
    CFX_CUDA(cudaMemsetAsync(p->state, 0, (size_t)p->L * p->n * p->H * sizeof(float), st));
    return CFX_OK;
}

int cfx_policy_set_step(cfx_policy* p, uint64_t step, void* stream) {
    CFX_REQUIRE(p, "cfx_policy_set_step: NULL handle");
    CFX_GUARD(p->device);
    cudaStream_t st = stream ? (cudaStream_t)stream : p->stream;
    unsigned long long v = step;
    CFX_CUDA(cudaMemcpyAsync(p->step_ctr, &v, sizeof(v), cudaMemcpyHostToDevice, st));
    CFX_CUDA(cudaStreamSynchronize(st));
    return CFX_OK;
}

int cfx_policy_get_step(cfx_policy* p, uint64_t* step) {
    CFX_REQUIRE(p && step, "cfx_policy_get_step: NULL argument");
    CFX_GUARD(p->device);
    unsigned long long v = 0;
    CFX_CUDA(cudaMemcpyAsync(&v, p->step_ctr, sizeof(v), cudaMemcpyDeviceToHost, p->stream));
    CFX_CUDA(cudaStreamSynchronize(p->stream));
    *step = v;
    return CFX_OK;
}

int cfx_policy_bump_step(cfx_policy* p, void* stream) {
    CFX_REQUIRE(p, "cfx_policy_bump_step: NULL handle");
    CFX_GUARD(p->device);
    return launch_bump(p->step_ctr, stream ? (cudaStream_t)stream : p->stream);
}

void* cfx_policy_stream(cfx_policy* p) { return p ? (void*)p->stream : nullptr; }
int cfx_policy_last_launches(const cfx_policy* p) { return p ? p->last_launches : 0; }

// ------------------------------------------------------------------ forward
// One forward over the 128-env tiles [tile_begin, tile_end) of the batch (tile_end = 0: all;
// slices are a fused-kernel feature, used by the pipelined host-buffer forward).
static int forward_range(cfx_policy* p, const cfx_forward_io* io, void* stream, int tile_begin, int tile_end) {
    CFX_REQUIRE(p && io, "cfx_policy_forward: NULL argument");
    CFX_REQUIRE(io->records != nullptr, "cfx_policy_forward: records is NULL");
    CFX_REQUIRE(((uintptr_t)io->records & 15) == 0, "cfx_policy_forward: records not 16-byte aligned");
    CFX_REQUIRE(io->actions != nullptr, "cfx_policy_forward: actions is NULL");
    CFX_GUARD(p->device);
    cudaStream_t st = stream ? (cudaStream_t)stream : p->stream;
    int launches = 0, rc;
    if (p->precision == CFX_PREC_FP32) {
        StrictArgs a;
        a.n = p->n; a.H = p->H; a.L = p->L; a.A = p->A;
        a.game = p->game;
        a.params = p->params;
        a.gates_t = p->gates_t;
        a.records = io->records;
        a.prev_terminals = io->prev_terminals;
        a.uniforms = io->uniforms;
        a.state = p->state;
        a.scratch_h[0] = p->scratch_h[0];
        a.scratch_h[1] = p->scratch_h[1];
        a.logits_av = io->logits_av ? io->logits_av : p->logits_scratch;
        a.r_state = io->r_state;
        a.r_state_bf16 = io->r_state_bf16 ? 1 : 0;
        a.env_actions = io->env_actions;
        a.actions = io->actions;
        a.logprobs = io->logprobs;
        a.values = io->values;
        a.seed = io->seed;
        a.env_offset = io->env_offset;
        a.step_ctr = p->step_ctr;
        rc = strict_forward(a, st, &launches);
    } else {
        CFX_REQUIRE(p->fused != nullptr, "cfx_policy_forward: fused plan missing");
        FusedArgs a;
        a.records = io->records;
        a.prev_terminals = io->prev_terminals;
        a.uniforms = io->uniforms;
        a.state = p->state;
        a.env_actions = io->env_actions;
        a.actions = io->actions;
        a.logprobs = io->logprobs;
        a.values = io->values;
        a.logits_av = io->logits_av;
        a.r_state = io->r_state;
        a.r_state_bf16 = io->r_state_bf16 ? 1 : 0;
        a.seed = io->seed;
        a.env_offset = io->env_offset;
        a.step_ctr = p->step_ctr;
        a.bump_step = io->bump_step ? 1 : 0;   // folded into the kernel: no extra launch
        a.tile_begin = tile_begin;
        a.tile_end = tile_end;
        rc = fused_forward(p->fused, a, st, &launches);
    }
    if (rc) return rc;
    if (io->bump_step && p->precision == CFX_PREC_FP32) {
        rc = launch_bump(p->step_ctr, st);
        if (rc) return rc;
        launches++;
    }
    p->last_launches = launches;
    return CFX_OK;
}

int cfx_policy_forward(cfx_policy* p, const cfx_forward_io* io, void* stream) {
    return forward_range(p, io, stream, 0, 0);
}

}  // extern "C"

extern "C" int cfx_policy_check(cfx_policy* p, void* stream) {
    CFX_REQUIRE(p, "cfx_policy_check: NULL handle");
    CFX_GUARD(p->device);
    cudaStream_t st = stream ? (cudaStream_t)stream : p->stream;
    CFX_CUDA(cudaStreamSynchronize(st));
    if (p->fused) {
        unsigned status = 0;
        int rc = fused_check_status(p->fused, st, &status);
        if (rc) return rc;
        if (status) {
            set_error("device-side wait timed out: site %u, block %u", status & 0xFF, status >> 8);
            return CFX_ERR_DEVICE_TIMEOUT;
        }
    }
    return CFX_OK;
}

extern "C" int cfx_selftest_wait_timeout(int device, unsigned limit_ms) {
    CFX_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, "cfx_selftest_wait_timeout: limit_ms=%u out of [1,1000]", limit_ms);
    CFX_GUARD(device);
    unsigned status = 0;
    int rc = fused_selftest_wait_timeout(limit_ms, &status);
    if (rc) return rc;
    if (status == 0) {
        set_error("self-test: the bounded wait did not report a timeout");
        return CFX_ERR_CUDA;
    }
    set_error("device-side wait timed out: site %u, block %u (self-test)", status & 0xFF, status >> 8);
    return CFX_ERR_DEVICE_TIMEOUT;
}

// ------------------------------------------------------------------ host-buffer forward
template <typename T>
static int ensure_staging(T** slot, size_t count) {
    if (*slot) return CFX_OK;
    CFX_CUDA(cudaMalloc((void**)slot, count * sizeof(T)));
    return CFX_OK;
}

extern "C" {

int cfx_policy_forward_host(cfx_policy* p, const cfx_forward_io* h) {
    CFX_REQUIRE(p && h, "cfx_policy_forward_host: NULL argument");
    CFX_REQUIRE(h->records && h->actions, "cfx_policy_forward_host: records/actions is NULL");
    CFX_GUARD(p->device);
    cudaStream_t st = p->stream;
    const size_t n = (size_t)p->n;
    // r_state staging in floats: bf16 records take half
    const size_t lav = n * (size_t)(p->A + 1), rs = (size_t)p->L * n * p->H / (h->r_state_bf16 ? 2 : 1);
    int rc;
    if ((rc = ensure_staging(&p->st_records, n * (size_t)p->rec_bytes))) return rc;
    if ((rc = ensure_staging(&p->st_actions, n))) return rc;
    if (h->prev_terminals && (rc = ensure_staging(&p->st_terminals, n))) return rc;
    if (h->uniforms && (rc = ensure_staging(&p->st_uniforms, n))) return rc;
    if (h->env_actions && (rc = ensure_staging(&p->st_env_actions, n))) return rc;
    if (h->logprobs && (rc = ensure_staging(&p->st_logprobs, n))) return rc;
    if (h->values && (rc = ensure_staging(&p->st_values, n))) return rc;
    if (h->logits_av && (rc = ensure_staging(&p->st_logits, lav))) return rc;
    if (h->r_state && (rc = ensure_staging(&p->st_r_state, (size_t)p->L * n * p->H))) return rc;

    cfx_forward_io d = *h;
    d.records = p->st_records;
    d.prev_terminals = h->prev_terminals ? p->st_terminals : nullptr;
    d.uniforms = h->uniforms ? p->st_uniforms : nullptr;
    d.env_actions = h->env_actions ? p->st_env_actions : nullptr;
    d.actions = p->st_actions;
    d.logprobs = h->logprobs ? p->st_logprobs : nullptr;
    d.values = h->values ? p->st_values : nullptr;
    d.logits_av = h->logits_av ? p->st_logits : nullptr;
    d.r_state = h->r_state ? p->st_r_state : nullptr;

    // The record upload dominates a host-buffer step (996 bytes per env over PCIe against
    // ~1.6 ns of kernel time).  With the fused kernel and a large batch the records go up in
    // slices on a copy stream and the kernel runs slice by slice behind them (a launch takes a
    // tile range), so that only the last slice's kernel is not hidden under the upload.
    const int tiles = (int)((n + 127) / 128);
    int slices = 1;
    if (p->precision != CFX_PREC_FP32) {
        slices = (int)(n / kHostSliceEnvs);
        slices = slices < 1 ? 1 : (slices > kHostSlicesMax ? kHostSlicesMax : slices);
    }
    if (slices == 1) {
        CFX_CUDA(cudaMemcpyAsync(p->st_records, h->records, n * (size_t)p->rec_bytes, cudaMemcpyHostToDevice, st));
        if (h->prev_terminals)
            CFX_CUDA(cudaMemcpyAsync(p->st_terminals, h->prev_terminals, n * sizeof(float),
                                     cudaMemcpyHostToDevice, st));
        if (h->uniforms)
            CFX_CUDA(cudaMemcpyAsync(p->st_uniforms, h->uniforms, n * sizeof(float),
                                     cudaMemcpyHostToDevice, st));
        rc = cfx_policy_forward(p, &d, st);
        if (rc) return rc;
    } else {
        if (!p->copy_stream) {
            CFX_CUDA(cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
            CFX_CUDA(cudaEventCreateWithFlags(&p->host_fence, cudaEventDisableTiming));
            for (int i = 0; i < kHostSlicesMax; i++)
                CFX_CUDA(cudaEventCreateWithFlags(&p->slice_ready[i], cudaEventDisableTiming));
        }
        cudaStream_t cs = p->copy_stream;
        // the staging buffers may still be read by work queued earlier on the handle's stream
        CFX_CUDA(cudaEventRecord(p->host_fence, st));
        CFX_CUDA(cudaStreamWaitEvent(cs, p->host_fence, 0));
        if (h->prev_terminals)
            CFX_CUDA(cudaMemcpyAsync(p->st_terminals, h->prev_terminals, n * sizeof(float),
                                     cudaMemcpyHostToDevice, cs));
        if (h->uniforms)
            CFX_CUDA(cudaMemcpyAsync(p->st_uniforms, h->uniforms, n * sizeof(float),
                                     cudaMemcpyHostToDevice, cs));
        int per = (tiles + slices - 1) / slices;
        per += per & 1;   // slices start at even tiles (CTA pairs)
        int launches = 0;
        for (int k = 0, t0 = 0; t0 < tiles; k++, t0 += per) {
            const int t1 = t0 + per < tiles ? t0 + per : tiles;
            const size_t e0 = (size_t)t0 * 128, e1 = (size_t)t1 * 128 < n ? (size_t)t1 * 128 : n;
            CFX_CUDA(cudaMemcpyAsync(p->st_records + e0 * p->rec_bytes, h->records + e0 * p->rec_bytes,
                                     (e1 - e0) * (size_t)p->rec_bytes, cudaMemcpyHostToDevice, cs));
            CFX_CUDA(cudaEventRecord(p->slice_ready[k], cs));
            CFX_CUDA(cudaStreamWaitEvent(st, p->slice_ready[k], 0));
            cfx_forward_io dk = d;
            dk.bump_step = (t1 == tiles) ? h->bump_step : 0;   // the last slice bumps the counter
            rc = forward_range(p, &dk, st, t0, t1);
            if (rc) return rc;
            launches += p->last_launches;
        }
        p->last_launches = launches;
    }
    CFX_CUDA(cudaMemcpyAsync(h->actions, p->st_actions, n * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    if (h->env_actions)
        CFX_CUDA(cudaMemcpyAsync(h->env_actions, p->st_env_actions, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (h->logprobs)
        CFX_CUDA(cudaMemcpyAsync(h->logprobs, p->st_logprobs, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (h->values)
        CFX_CUDA(cudaMemcpyAsync(h->values, p->st_values, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (h->logits_av)
        CFX_CUDA(cudaMemcpyAsync(h->logits_av, p->st_logits, lav * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (h->r_state)
        CFX_CUDA(cudaMemcpyAsync(h->r_state, p->st_r_state, rs * sizeof(float), cudaMemcpyDeviceToHost, st));
    return cfx_policy_check(p, st);
}

// ------------------------------------------------------------------ stand-alone stages
int cfx_expand_obs(int device, const uint8_t* records, float* features, int n, void* stream) {
    CFX_REQUIRE(records && features && n > 0, "cfx_expand_obs: bad argument");
    // the 51 tail floats of a record are read as 32-bit words
    CFX_REQUIRE(((uintptr_t)records & 3) == 0, "cfx_expand_obs: records not 4-byte aligned");
    CFX_GUARD(device);
    return launch_expand(records, features, n, (cudaStream_t)stream);
}

int cfx_sample_actions(int device, const float* logits, int ld, int num_actions,
                       const float* uniforms, int n, int32_t* actions, float* logprobs,
                       void* stream) {
    CFX_REQUIRE(logits && uniforms && actions && logprobs && n > 0, "cfx_sample_actions: bad argument");
    CFX_REQUIRE(num_actions >= 2 && num_actions <= kMaxActions && ld >= num_actions,
                "cfx_sample_actions: num_actions=%d ld=%d", num_actions, ld);
    CFX_GUARD(device);
    return launch_sample(logits, ld, num_actions, uniforms, 0, 0, nullptr, n, nullptr, actions,
                         logprobs, nullptr, (cudaStream_t)stream);
}

int cfx_philox_uniforms(int device, uint64_t seed, uint64_t env_offset, uint64_t step, int n,
                        float* uniforms, void* stream) {
    CFX_REQUIRE(uniforms && n > 0, "cfx_philox_uniforms: bad argument");
    CFX_GUARD(device);
    return launch_uniforms(seed, env_offset, step, n, uniforms, (cudaStream_t)stream);
}

// ------------------------------------------------------------------ helpers
int cfx_device_count(int* count) {
    CFX_REQUIRE(count, "cfx_device_count: NULL");
    *count = 0;
    CFX_CUDA(cudaGetDeviceCount(count));
    return CFX_OK;
}

int cfx_device_name(int device, char* buf, size_t len, int* sm_count, int* cc_major, int* cc_minor) {
    cudaDeviceProp prop;
    CFX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (buf && len) {
        strncpy(buf, prop.name, len - 1);
        buf[len - 1] = 0;
    }
    if (sm_count) *sm_count = prop.multiProcessorCount;
    if (cc_major) *cc_major = prop.major;
    if (cc_minor) *cc_minor = prop.minor;
    return CFX_OK;
}

int cfx_device_alloc(int device, void** ptr, size_t bytes) {
    CFX_REQUIRE(ptr, "cfx_device_alloc: NULL");
    CFX_GUARD(device);
    CFX_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
    return CFX_OK;
}

int cfx_device_free(int device, void* ptr) {
    CFX_GUARD(device);
    CFX_CUDA(cudaFree(ptr));
    return CFX_OK;
}

int cfx_host_alloc_pinned(void** ptr, size_t bytes) {
    CFX_REQUIRE(ptr, "cfx_host_alloc_pinned: NULL");
    CFX_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1));
    return CFX_OK;
}

int cfx_host_free_pinned(void* ptr) {
    CFX_CUDA(cudaFreeHost(ptr));
    return CFX_OK;
}

int cfx_memcpy_h2d(int device, void* dst, const void* src, size_t bytes, void* stream) {
    CFX_GUARD(device);
    CFX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return CFX_OK;
}

int cfx_memcpy_d2h(int device, void* dst, const void* src, size_t bytes, void* stream) {
    CFX_GUARD(device);
    CFX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return CFX_OK;
}

int cfx_memset(int device, void* dst, int value, size_t bytes, void* stream) {
    CFX_GUARD(device);
    CFX_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return CFX_OK;
}

int cfx_stream_sync(int device, void* stream) {
    CFX_GUARD(device);
    CFX_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return CFX_OK;
}

struct cfx_timer {
    int device;
    cudaEvent_t a, b;
};

int cfx_timer_create(int device, void** timer) {
    CFX_REQUIRE(timer, "cfx_timer_create: NULL");
    CFX_GUARD(device);
    cfx_timer* t = new (std::nothrow) cfx_timer();
    CFX_REQUIRE(t, "cfx_timer_create: out of host memory");
    t->device = device;
    CFX_CUDA(cudaEventCreate(&t->a));
    CFX_CUDA(cudaEventCreate(&t->b));
    *timer = t;
    return CFX_OK;
}

int cfx_timer_destroy(void* timer) {
    cfx_timer* t = (cfx_timer*)timer;
    if (!t) return CFX_OK;
    DeviceGuard g(t->device);
    cudaEventDestroy(t->a);
    cudaEventDestroy(t->b);
    delete t;
    return CFX_OK;
}

int cfx_timer_start(void* timer, void* stream) {
    cfx_timer* t = (cfx_timer*)timer;
    CFX_REQUIRE(t, "cfx_timer_start: NULL");
    CFX_GUARD(t->device);
    CFX_CUDA(cudaEventRecord(t->a, (cudaStream_t)stream));
    return CFX_OK;
}

int cfx_timer_stop(void* timer, void* stream) {
    cfx_timer* t = (cfx_timer*)timer;
    CFX_REQUIRE(t, "cfx_timer_stop: NULL");
    CFX_GUARD(t->device);
    CFX_CUDA(cudaEventRecord(t->b, (cudaStream_t)stream));
    return CFX_OK;
}

int cfx_timer_elapsed_ms(void* timer, float* ms) {
    cfx_timer* t = (cfx_timer*)timer;
    CFX_REQUIRE(t && ms, "cfx_timer_elapsed_ms: NULL");
    CFX_GUARD(t->device);
    CFX_CUDA(cudaEventSynchronize(t->b));
    CFX_CUDA(cudaEventElapsedTime(ms, t->a, t->b));
    return CFX_OK;
}

}  // extern "C"
