// Shared definitions of the B200 policy-forward library: constants of the
// record / arena layout, the handle, error plumbing.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include "../../include/cfx.h"

namespace cfx {

constexpr int kObs = CFX_OBS_FEATURES;   // 843 features
constexpr int kMap = CFX_OBS_MAP;        // 792 one-byte map features
constexpr int kTail = CFX_OBS_TAIL;      // 51 raw fp32 tail features
constexpr int kRec = CFX_RECORD_BYTES;   // 996-byte record
constexpr int kMaxActions = 63;
// classic game (reference craftax_classic.cu:38-59): 148-byte record, 1345 features
constexpr int kClassicRec = CFX_CLASSIC_RECORD_BYTES, kClassicObs = CFX_CLASSIC_OBS_FEATURES;
constexpr int kClassicCells = 63, kClassicBlocks = 17, kClassicInv = 12;

// Arena offsets in floats (reference order, craftax_full.cu:9094-9102).
struct ArenaLayout {
    size_t w_enc, b_enc, w_gru, w_a, b_a, w_v, b_v, count;
    __host__ __device__ static ArenaLayout make(int H, int L, int A, int obs = kObs) {
        ArenaLayout o;
        o.w_enc = 0;
        o.b_enc = (size_t)obs * H;
        o.w_gru = o.b_enc + H;
        o.w_a = o.w_gru + (size_t)L * 3 * H * H;
        o.b_a = o.w_a + (size_t)A * H;
        o.w_v = o.b_a + A;
        o.b_v = o.w_v + H;
        o.count = o.b_v + 1;
        return o;
    }
};

// Thread-local error string behind cfx_last_error().
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define CFX_CUDA(call)                                                        \
    do {                                                                      \
        cudaError_t _e = (call);                                              \
        if (_e != cudaSuccess) return ::cfx::cuda_fail(_e, #call, __FILE__, __LINE__); \
    } while (0)

#define CFX_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) {                         \
            ::cfx::set_error(__VA_ARGS__);     \
            return CFX_ERR_INVALID;            \
        }                                      \
    } while (0)

// Scoped cudaSetDevice.  Entry points use CFX_GUARD, which returns an error when the device
// cannot be selected instead of carrying on with whatever device is current.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

#define CFX_GUARD(dev)                                                                   \
    ::cfx::DeviceGuard _cfx_guard(dev);                                                  \
    do {                                                                                 \
        if (!_cfx_guard.ok) {                                                            \
            cudaGetLastError();                                                          \
            ::cfx::set_error("%s: cannot select CUDA device %d", __func__, (int)(dev));  \
            return CFX_ERR_CUDA;                                                         \
        }                                                                                \
    } while (0)

}  // namespace cfx
