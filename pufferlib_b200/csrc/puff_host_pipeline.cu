// Host-buffer entry point: the advantage op for a caller that holds its
// experience buffers in host memory.
//
// Stands where the reference's host-tensor route stands (the Python wrapper's
// `.cpu()` branch, pufferlib/pufferl.py:666-678, feeding
// compute_puff_advantage_cpu, pufferlib/extensions/pufferlib.cpp:75-85).  Rows
// are independent, so the buffer is cut into row blocks that flow through a
// ring of device slots: four host->device copies, one kernel, one
// device->host copy per block, each slot on its own stream, so uploads,
// kernels and downloads of neighbouring blocks overlap and both PCIe
// directions stay busy.  The download is a pitched copy of H-1 columns: the
// caller's advantages[:, H-1] is never written, like the device op.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>

#include "../../include/puff_advantage.h"

namespace puff {
int take_device_status();   // puff_advantage_sm100.cu

constexpr int kSlots = 3;
constexpr int kMaxDevices = 64;

struct HostPipe {
    std::mutex mu;
    bool ready = false;
    cudaStream_t stream[kSlots] = {};
    float* slab[kSlots] = {};          // 5 arrays of `cap_elems` floats + `cap_rows` floats
    size_t cap_elems = 0;
    size_t cap_rows = 0;
};
static HostPipe g_pipe[kMaxDevices];

static void pipe_free(HostPipe& p)
{
    for (int i = 0; i < kSlots; ++i) {
        if (p.slab[i] != nullptr) cudaFree(p.slab[i]);
        if (p.stream[i] != nullptr) cudaStreamDestroy(p.stream[i]);
        p.slab[i] = nullptr;
        p.stream[i] = nullptr;
    }
    p.cap_elems = p.cap_rows = 0;
    p.ready = false;
}

static cudaError_t pipe_reserve(HostPipe& p, size_t block_elems, size_t block_rows)
{
    if (p.ready && p.cap_elems >= block_elems && p.cap_rows >= block_rows) return cudaSuccess;
    pipe_free(p);
    for (int i = 0; i < kSlots; ++i) {
        cudaError_t e = cudaStreamCreateWithFlags(&p.stream[i], cudaStreamNonBlocking);
        if (e != cudaSuccess) return e;
        e = cudaMalloc(&p.slab[i], (5 * block_elems + block_rows) * sizeof(float));
        if (e != cudaSuccess) return e;
    }
    p.cap_elems = block_elems;
    p.cap_rows = block_rows;
    p.ready = true;
    return cudaSuccess;
}

static long long env_ll(const char* name, long long fallback)
{
    const char* s = getenv(name);
    if (s == nullptr || *s == '\0') return fallback;
    return atoll(s);
}
}  // namespace puff

using namespace puff;

static int host_pipeline(const float* h_values, const float* h_rewards, const float* h_dones,
                         const float* h_importance, float* h_advantages, float* h_seg_abs_sum,
                         float gamma, float lambda, float rho_clip, float c_clip,
                         long long num_segments, long long horizon, int variant, int device, bool compute)
{
    if (num_segments < 0 || horizon < 0) return PUFF_ERR_SHAPE;
    if (variant < PUFF_VARIANT_AUTO || variant > PUFF_VARIANT_GENERIC) return PUFF_ERR_VARIANT;
    if (device < 0 || device >= kMaxDevices) return PUFF_ERR_ARCH;
    if (num_segments == 0) return PUFF_OK;
    if (horizon < 2) {
        if (h_seg_abs_sum != nullptr)
            for (long long s = 0; s < num_segments; ++s) h_seg_abs_sum[s] = 0.0f;
        return PUFF_OK;
    }
    if (h_values == nullptr || h_rewards == nullptr || h_dones == nullptr || h_importance == nullptr ||
        h_advantages == nullptr)
        return PUFF_ERR_NULL;

    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return static_cast<int>(e);

    HostPipe& p = g_pipe[device];
    std::lock_guard<std::mutex> lock(p.mu);

    // row blocks of about PUFF_HOST_BLOCK_BYTES (default 16 MB, measured best of 4..32 MB) per array,
    // a multiple of 32 rows
    const long long target = env_ll("PUFF_HOST_BLOCK_BYTES", 16ll << 20);
    long long block_rows = target / (horizon * 4);
    block_rows = (block_rows / 32) * 32;
    if (block_rows < 32) block_rows = 32;
    if (block_rows > num_segments) block_rows = num_segments;
    // keep every array slot 256-byte aligned
    const size_t block_elems = (static_cast<size_t>(block_rows) * horizon + 63) & ~static_cast<size_t>(63);
    const size_t rows_cap = (static_cast<size_t>(block_rows) + 63) & ~static_cast<size_t>(63);

    int rc = PUFF_OK;
    e = pipe_reserve(p, block_elems, rows_cap);
    if (e != cudaSuccess) {
        rc = static_cast<int>(e);
    } else {
        int slot = 0;
        const float* h_in[4] = {h_values, h_rewards, h_dones, h_importance};
        // full blocks through the body; the last two blocks' worth of rows is cut into halves
        // of what remains, so that the kernel and the download that trail the last upload
        // are short (the uploads are what the wall time is made of)
        const long long min_rows = env_ll("PUFF_HOST_TAPER", 1) != 0 ? ((1ll << 20) / (horizon * 4) / 32 + 1) * 32 : block_rows;
        long long rows = 0;
        for (long long r0 = 0; r0 < num_segments && rc == PUFF_OK; r0 += rows, slot = (slot + 1) % kSlots) {
            const long long left = num_segments - r0;
            rows = block_rows;
            if (left <= 2 * block_rows && min_rows < block_rows) {
                rows = ((left / 2 + 31) / 32) * 32;
                if (rows < min_rows) rows = min_rows;
                if (rows > block_rows) rows = block_rows;
            }
            if (rows > left) rows = left;
            const size_t n = static_cast<size_t>(rows) * horizon;
            const size_t off = static_cast<size_t>(r0) * horizon;
            cudaStream_t st = p.stream[slot];
            float* d_in[4];
            for (int a = 0; a < 4; ++a) d_in[a] = p.slab[slot] + a * p.cap_elems;
            float* d_adv = p.slab[slot] + 4 * p.cap_elems;
            float* d_abs = h_seg_abs_sum != nullptr ? p.slab[slot] + 5 * p.cap_elems : nullptr;
            for (int a = 0; a < 4 && e == cudaSuccess; ++a)
                e = cudaMemcpyAsync(d_in[a], h_in[a] + off, n * sizeof(float), cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) { rc = static_cast<int>(e); break; }
            if (compute)
                rc = puff_advantage_sm100_launch(d_in[0], d_in[1], d_in[2], d_in[3], d_adv, d_abs, gamma, lambda,
                                                 rho_clip, c_clip, rows, horizon, variant, st);
            if (rc != PUFF_OK) break;
            e = cudaMemcpy2DAsync(h_advantages + off, horizon * sizeof(float), d_adv, horizon * sizeof(float),
                                  (horizon - 1) * sizeof(float), rows, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess && d_abs != nullptr)
                e = cudaMemcpyAsync(h_seg_abs_sum + r0, d_abs, rows * sizeof(float), cudaMemcpyDeviceToHost, st);
            if (e != cudaSuccess) rc = static_cast<int>(e);
        }
        for (int i = 0; i < kSlots; ++i) {
            cudaError_t es = cudaStreamSynchronize(p.stream[i]);
            if (es != cudaSuccess && rc == PUFF_OK) rc = static_cast<int>(es);
        }
        // every kernel of this call has finished: a bounded wait that gave up inside one of them
        // left part of the output unwritten, which must not be reported as success
        if (rc == PUFF_OK) rc = take_device_status();
    }
    cudaSetDevice(prev);
    return rc;
}

extern "C" int puff_advantage_sm100_host(const float* h_values, const float* h_rewards, const float* h_dones,
                                         const float* h_importance, float* h_advantages, float* h_seg_abs_sum,
                                         float gamma, float lambda, float rho_clip, float c_clip,
                                         long long num_segments, long long horizon, int variant, int device)
{
    return host_pipeline(h_values, h_rewards, h_dones, h_importance, h_advantages, h_seg_abs_sum, gamma, lambda,
                         rho_clip, c_clip, num_segments, horizon, variant, device, true);
}

extern "C" int puff_advantage_sm100_host_copies_only(const float* h_values, const float* h_rewards,
                                                     const float* h_dones, const float* h_importance,
                                                     float* h_advantages, float* h_seg_abs_sum,
                                                     long long num_segments, long long horizon, int device)
{
    return host_pipeline(h_values, h_rewards, h_dones, h_importance, h_advantages, h_seg_abs_sum, 0.f, 0.f, 0.f, 0.f,
                         num_segments, horizon, PUFF_VARIANT_AUTO, device, false);
}

extern "C" int puff_advantage_sm100_host_release(int device)
{
    if (device < 0 || device >= kMaxDevices) return PUFF_ERR_ARCH;
    HostPipe& p = g_pipe[device];
    std::lock_guard<std::mutex> lock(p.mu);
    if (!p.ready) return PUFF_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    pipe_free(p);
    cudaSetDevice(prev);
    return PUFF_OK;
}
