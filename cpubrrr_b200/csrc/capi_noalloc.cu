// Router entry point for callers that must not allocate device memory.
//
// Who needs it: a serving host that has already handed every free byte of HBM to its own pools
// (KV cache, weight arenas) has nothing left for cudaMalloc to return, and a request path that
// runs while other streams are busy cannot afford cudaMalloc / cudaFree at all, because both
// take the driver's allocation lock and cudaFree synchronises the whole device.  The ordinary
// brrr_router_topk allocates a temporary for the re-tiled router matrix on every call; this
// variant keeps that temporary, and the CTA arrival counter, in a fixed array that is part of
// the library image, so a call performs no allocation of any kind.
#include "../../include/brrr.h"
#include "brrr_kernels.h"

using namespace brrr;

namespace {

// Largest router this entry point accepts.
constexpr int NA_MAX_EXPERTS = 128;
constexpr int NA_MAX_D = 4096;
constexpr size_t NA_TILED_FLOATS = (size_t)(NA_MAX_EXPERTS / 32) * (NA_MAX_D / RT_TJ) * RT_TILE_FLOATS;
constexpr size_t NA_COUNTER_BYTES = 256;                                                                  // keeps the matrix 256-byte aligned
constexpr size_t NA_SCRATCH_BYTES = NA_COUNTER_BYTES + NA_TILED_FLOATS * sizeof(float);                   // about 2.1 MB

// Every GPU that loads the library holds this array until the process exits.
static __device__ __align__(256) unsigned char g_router_scratch[NA_SCRATCH_BYTES];

// In host code the name above is only a stand-in for the symbol; the device address has to be
// asked for, once per device, with that device current.
unsigned char *g_scratch_addr[64] = {nullptr};

int scratch_for_current_device(unsigned char **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BRRR_ERR_CUDA;
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_router_scratch) != cudaSuccess || !p) return BRRR_ERR_CUDA;
        g_scratch_addr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_scratch_addr[dev];
    return BRRR_OK;
}

}  // namespace

extern "C" int brrr_router_topk_noalloc(const float *d_w, const float *d_b, const float *d_xn, int ne, int d, int topk,
                                        float *d_logits, int32_t *d_top, float *d_wts, void *stream) {
    if (!d_w || !d_xn || !d_logits || !d_top || !d_wts || ne <= 0 || d <= 0 || d % 64 || topk <= 0 || topk > 8 || topk > ne) return BRRR_ERR_ARG;
    if (ne > NA_MAX_EXPERTS || d > NA_MAX_D) return BRRR_ERR_RANGE;      // larger than the built-in scratch
    unsigned char *scratch = nullptr;
    int s = scratch_for_current_device(&scratch);
    if (s != BRRR_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned int *counter = reinterpret_cast<unsigned int *>(scratch);
    float *tiled = reinterpret_cast<float *>(scratch + NA_COUNTER_BYTES);
    // The array keeps whatever the previous call left: the arrival counter must start at zero,
    // and the tiled matrix is rewritten in full (padding included) for this call's shape.
    if (cudaMemsetAsync(counter, 0, sizeof(unsigned int), st) != cudaSuccess) return BRRR_ERR_CUDA;
    launch_router_pack(d_w, ne, d, tiled, st);
    if (launch_ffn_in(d_xn, nullptr, 0.0f, d, tiled, d_b, ne, topk, d_logits, d_top, d_wts, counter, nullptr, false, st) != cudaSuccess) return BRRR_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? BRRR_OK : BRRR_ERR_CUDA;
}
