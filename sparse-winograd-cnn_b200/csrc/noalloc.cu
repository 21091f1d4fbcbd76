// Weight-gradient entry point for callers that cannot allocate device memory.
//
// wg2x2_conv_bwd needs scratch memory for dW whenever the contraction over the P tiles is split
// across CTAs, and asks the caller to allocate it.  Some callers cannot: code running inside a
// framework hook that only hands out the op's inputs and outputs, a real-time or safety-reviewed
// process that forbids cudaMalloc after start-up, or a plug-in running while the host application
// has reserved all device memory.  For them the scratch lives in a fixed array inside this
// library: kMaxScratchFloats floats (32 MiB) of global memory on every GPU that loads the
// library, held until the process exits.
#include <mutex>

#include "wg_common.cuh"

namespace wg {
int conv_dw_splits(long long P, int C, int K);
int conv_dw_ffma(const float *V, const float *dY, const float *mask, float *dW, int B, int H, int W, int C, int K, int layout,
                 float *scratch, int splits, cudaStream_t st);

constexpr size_t kMaxScratchFloats = (size_t)8 << 20;  // 8 Mi floats = 32 MiB
static __device__ __align__(256) float g_dw_scratch[kMaxScratchFloats];

// In host code `g_dw_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
constexpr int kMaxDevices = 64;
static float *g_scratch_ptr[kMaxDevices];
static std::mutex g_scratch_mutex;

static float *scratch_for_current_device()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dw_scratch) != cudaSuccess) return nullptr;
        g_scratch_ptr[dev] = static_cast<float *>(p);
    }
    return g_scratch_ptr[dev];
}
}  // namespace wg

extern "C" {

size_t wg2x2_conv_bwd_dw_noalloc_max_bytes(void) { return wg::kMaxScratchFloats * sizeof(float); }

int wg2x2_conv_bwd_dw_noalloc(const float *V, const float *dY, const float *mask, float *dW, int B, int H, int W, int C, int K,
                              int layout, void *stream)
{
    if (!V || !dY || !dW || B <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0) return WG2X2_ERR_BAD_ARG;
    if (layout != WG2X2_NHWC && layout != WG2X2_NCHW) return WG2X2_ERR_BAD_ARG;
    const long long P = (long long)B * ((H + 1) / 2) * ((W + 1) / 2);
    // same split count as wg2x2_conv_bwd, so the two entry points add in the same order
    const int splits = wg::conv_dw_splits(P, C, K);
    const size_t need = splits > 1 ? (size_t)splits * 16 * C * K : 0;
    if (need > wg::kMaxScratchFloats) return WG2X2_ERR_WORKSPACE;  // beyond the built-in scratch: use wg2x2_conv_bwd
    float *scratch = nullptr;
    if (need) {
        scratch = wg::scratch_for_current_device();
        if (!scratch) return WG2X2_ERR_LAUNCH;
    }
    return wg::conv_dw_ffma(V, dY, mask, dW, B, H, W, C, K, layout, scratch, splits, (cudaStream_t)stream);
}

}  // extern "C"
