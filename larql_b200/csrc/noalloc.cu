// lq_q4k_matvec_static — a Q4_K matvec entry point that allocates nothing.
//
// Who needs it: hosts that must not call cudaMalloc while they run.  Typical cases are a
// serving process that has handed every free byte of HBM to its own pools (weights, KV
// cache) at start-up, so a later cudaMalloc from a library would fail or evict; a plugin
// living under a framework allocator that forbids raw device allocations; and latency-
// critical loops that cannot afford the implicit device-wide synchronisation cudaMalloc and
// cudaFree bring.  The regular entry points grow a per-context workspace on first use; this
// one never does.
//
// The matvec needs scratch beyond its inputs and output: the prepared copy of the activation
// (f32 vector, two fixed-point byte planes, per-block step / sum / |sum|) that the scan kernel
// reads.  Here that scratch is a fixed array in the library's device image,
// LQ_STATIC_SCRATCH_BYTES (128 KiB) per GPU that loads the library, held until the process
// exits.  It bounds the problem: hidden <= LQ_STATIC_MAX_HIDDEN (16384); larger is refused.
//
// In host code the array's NAME is only a host-side handle, never a device address, so the
// address is fetched once per device with cudaGetSymbolAddress (with that device current) and
// that pointer is what the kernels get.  The first call on a device does this set-up; make
// that first call outside any stream capture.
//
// All calls on a device share the one array and it keeps the last call's contents.  The only
// part that must start clean is the error word, which every call clears; everything else is
// fully rewritten before it is read.  Two calls that overlap on the same GPU (different
// streams or threads) race on the scratch: serialise them.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/larql_cuda.h"
#include "kernels.h"

#define LQ_STATIC_MAX_HIDDEN 16384
#define LQ_STATIC_SCRATCH_BYTES (128 * 1024)

static __device__ __align__(256) unsigned char lq_static_scratch[LQ_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device
int g_sm_count[kMaxDevices] = {};

int say(char* errbuf, size_t errcap, int code, const char* msg, const char* detail = "") {
    if (errbuf && errcap) snprintf(errbuf, errcap, "%s%s", msg, detail);
    return code;
}

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" int lq_q4k_matvec_static(const uint8_t* w, size_t w_len, const float* x, size_t num_rows, size_t hidden,
                                    float* out, void* stream, char* errbuf, size_t errcap) {
    if (errbuf && errcap) errbuf[0] = 0;
    if (hidden % 256 != 0 || w_len < num_rows * (hidden / 256) * 144)
        return say(errbuf, errcap, LQ_REFUSED_SHAPE, "q4k_matvec_static: hidden % 256 != 0 or weights too short");
    if (hidden > LQ_STATIC_MAX_HIDDEN)
        return say(errbuf, errcap, LQ_REFUSED_UNSUPPORTED,
                   "q4k_matvec_static: hidden exceeds the static scratch (max 16384 columns)");
    if (num_rows == 0) return LQ_OK;
    if (num_rows > 0x7fffffffu) return say(errbuf, errcap, LQ_REFUSED_UNSUPPORTED, "q4k_matvec_static: too many rows");
    if (!w || !x || !out) return say(errbuf, errcap, LQ_ERR_ARGUMENT, "q4k_matvec_static: null pointer");
    if (((uintptr_t)w & 15) != 0) return say(errbuf, errcap, LQ_ERR_ARGUMENT, "q4k_matvec_static: weights not 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (hidden == 0) {
        cudaError_t e = cudaMemsetAsync(out, 0, num_rows * 4, st);
        return e == cudaSuccess ? LQ_OK : say(errbuf, errcap, LQ_ERR_CUDA, "memset: ", cudaGetErrorString(e));
    }

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return say(errbuf, errcap, LQ_ERR_CUDA, "cudaGetDevice: ", cudaGetErrorString(e));
    unsigned char* base = nullptr;
    int sms = 0;
    {
        // Set-up, once per device, with that device current: turn the symbol into a device address.
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, lq_static_scratch);
            if (e != cudaSuccess || !p)
                return say(errbuf, errcap, LQ_ERR_CUDA, "cudaGetSymbolAddress(lq_static_scratch): ", cudaGetErrorString(e));
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || n <= 0)
                return say(errbuf, errcap, LQ_ERR_CUDA, "cudaDeviceGetAttribute: ", cudaGetErrorString(e));
            g_sm_count[dev] = n;
            g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
        }
        base = g_scratch_ptr[dev];
        sms = g_sm_count[dev];
    }

    // Carve the array: [error word | xn | plane a | plane b | step | sum | abs], 256-byte pieces.
    const size_t H = hidden;
    unsigned char* p = base;
    int* err = reinterpret_cast<int*>(p);                     p += 256;
    float* xn = reinterpret_cast<float*>(p);                  p += up256(H * 4);
    uint32_t* xa = reinterpret_cast<uint32_t*>(p);            p += up256(H);
    uint32_t* xb = reinterpret_cast<uint32_t*>(p);            p += up256(H);
    float* bscale = reinterpret_cast<float*>(p);              p += up256(H / 32 * 4);
    float* bsum = reinterpret_cast<float*>(p);                p += up256(H / 32 * 4);
    float* babs = reinterpret_cast<float*>(p);                p += up256(H / 32 * 4);
    if (static_cast<size_t>(p - base) > LQ_STATIC_SCRATCH_BYTES)
        return say(errbuf, errcap, LQ_REFUSED_UNSUPPORTED, "q4k_matvec_static: scratch layout exceeds the array");

    // The error word is the one piece that must start at zero; the rest is rewritten by prep.
    e = cudaMemsetAsync(err, 0, 256, st);
    if (e != cudaSuccess) return say(errbuf, errcap, LQ_ERR_CUDA, "memset: ", cudaGetErrorString(e));
    lq::launch_prep(x, 1, (int)hidden, 0, 0.0, xn, xa, xb, bscale, bsum, babs, 0, nullptr, st);
    e = cudaGetLastError();
    if (e != cudaSuccess) return say(errbuf, errcap, LQ_ERR_CUDA, "prep launch: ", cudaGetErrorString(e));
    const lq::Q4kMat m{w, (int)num_rows, (int)hidden};
    const lq::XPrep xp{xn, xa, xb, bscale, bsum, babs};
    e = lq::launch_scan_q4k(m, xp, out, nullptr, nullptr, 0.0f, err, sms, st);
    if (e != cudaSuccess) return say(errbuf, errcap, LQ_ERR_CUDA, "scan launch: ", cudaGetErrorString(e));
    // Wait and report: the call is complete when it returns.
    int h_err = 0;
    e = cudaMemcpyAsync(&h_err, err, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return say(errbuf, errcap, LQ_ERR_CUDA, "synchronize: ", cudaGetErrorString(e));
    if (h_err == lq::DEV_ERR_TMA_TIMEOUT) return say(errbuf, errcap, LQ_ERR_TIMEOUT, "a bounded device-side wait ran out");
    if (h_err != 0) return say(errbuf, errcap, LQ_ERR_CUDA, "device-side error");
    return LQ_OK;
}
