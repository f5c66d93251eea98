// One small matrix per head:  out[i, h, :] = W[h] in[i, h, :]  (W [heads, n_out, n_in]), optionally times
// sigmoid(gate[i, h]).  This is how a latent attention folds its per-head key up-projection into the
// queries (W[h] = W_uk[h]^T, so that scores are taken against the cached latent itself) and expands the
// attended latent into the head's values (W[h] = W_uv[h]).  Head h's input starts at column in_off + h *
// in_stride of its row, its output at out_off + h * out_stride.
//
// CUDA cores, float32 accumulation over k in order, for both dtypes: a block takes HL_TOKENS tokens of one head,
// keeps their inputs in shared memory, and every thread owns output columns for all of those tokens.
#include "common.cuh"

namespace {

constexpr int HL_TOKENS = 16;
constexpr int HL_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(HL_THREADS)
head_linear_kernel(const T* __restrict__ in, long long ld_in, int in_off, int in_stride, const T* __restrict__ w,
                   T* __restrict__ out, long long ld_out, int out_off, int out_stride, int n, int n_in, int n_out,
                   const T* __restrict__ gate, long long ld_gate) {
  extern __shared__ float in_s[];                    // [HL_TOKENS][n_in]
  __shared__ float gate_s[HL_TOKENS];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.y;
  const int first = blockIdx.x * HL_TOKENS;
  const int count = min(HL_TOKENS, n - first);
  for (int e = threadIdx.x; e < HL_TOKENS * n_in; e += HL_THREADS) {
    const int t = e / n_in, k = e - t * n_in;
    in_s[e] = t < count ? to_f32<T>(in[(long long)(first + t) * ld_in + in_off + (long long)h * in_stride + k]) : 0.f;
  }
  if (threadIdx.x < HL_TOKENS) {
    float gv = 1.f;
    if (gate != nullptr && threadIdx.x < count)
      gv = 1.f / (1.f + expf(-to_f32<T>(gate[(long long)(first + threadIdx.x) * ld_gate + h])));
    gate_s[threadIdx.x] = gv;
  }
  __syncthreads();
  const T* wh = w + (long long)h * n_out * n_in;
  for (int o = threadIdx.x; o < n_out; o += HL_THREADS) {
    const T* wr = wh + (long long)o * n_in;
    float acc[HL_TOKENS];
#pragma unroll
    for (int t = 0; t < HL_TOKENS; ++t) acc[t] = 0.f;
    for (int k = 0; k < n_in; ++k) {
      const float wv = to_f32<T>(wr[k]);
#pragma unroll
      for (int t = 0; t < HL_TOKENS; ++t) acc[t] = fmaf(wv, in_s[t * n_in + k], acc[t]);
    }
#pragma unroll
    for (int t = 0; t < HL_TOKENS; ++t)
      if (t < count)
        out[(long long)(first + t) * ld_out + out_off + (long long)h * out_stride + o] = from_f32<T>(acc[t] * gate_s[t]);
  }
}

template <typename T>
int launch_head_linear(const void* in, long long ld_in, int in_off, int in_stride, const void* w, void* out, long long ld_out,
                       int out_off, int out_stride, int n, int heads, int n_in, int n_out, const void* gate,
                       long long ld_gate, cudaStream_t stream) {
  const size_t smem = (size_t)HL_TOKENS * n_in * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(head_linear_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "head_linear: %s", cudaGetErrorString(e));
  }
  hfee_launch(head_linear_kernel<T>, dim3((unsigned)((n + HL_TOKENS - 1) / HL_TOKENS), (unsigned)heads), dim3(HL_THREADS), smem,
              stream, (const T*)in, ld_in, in_off, in_stride, (const T*)w, (T*)out, ld_out, out_off, out_stride, n, n_in, n_out,
              (const T*)gate, ld_gate);
  return hfee_check_launch("head_linear");
}

}  // namespace

HFEE_API int hfee_head_linear(const void* in, long long ld_in, int in_off, int in_stride, const void* w, void* out,
                              long long ld_out, int out_off, int out_stride, int n, int heads, int n_in, int n_out,
                              const void* gate, long long ld_gate, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(heads > 0 && n_in > 0 && n_out > 0 && n_in <= 2048, "head_linear: bad sizes (n_in at most 2048)");
  if (dtype == HFEE_F32)
    return launch_head_linear<float>(in, ld_in, in_off, in_stride, w, out, ld_out, out_off, out_stride, n, heads, n_in, n_out, gate, ld_gate, stream);
  if (dtype == HFEE_BF16)
    return launch_head_linear<__nv_bfloat16>(in, ld_in, in_off, in_stride, w, out, ld_out, out_off, out_stride, n, heads, n_in, n_out, gate, ld_gate, stream);
  return hfee_fail(HFEE_ERR_ARG, "head_linear: unknown dtype %d", dtype);
}
