// One small matrix per head:  out[i, h, :] = W[h] in[i, h, :]  (W [heads, n_out, n_in]), optionally times
// sigmoid(gate[i, h]).  This is how a latent attention folds its per-head key up-projection into the
// queries (W[h] = W_uk[h]^T, so that scores are taken against the cached latent itself) and expands the
// attended latent into the head's values (W[h] = W_uv[h]).  Head h's input starts at column in_off + h *
// in_stride of its row, its output at out_off + h * out_stride.
//
// bfloat16 with 16-byte aligned head slices runs on the tensor cores (mma.sync.m16n8k16, float32 accumulation): a block
// takes 64 tokens x 64 output columns of one head, stages 64 columns of k of both operands in shared memory at a
// time, and each of its four warps owns 32 x 32 of the tile.  Everything else runs on the CUDA cores with float32
// accumulation over k in order: a block takes HL_TOKENS tokens of one head, keeps their inputs in shared memory,
// and every thread owns output columns for all of those tokens.
#include "mma_tiles.cuh"

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

constexpr int HM_TILE = 64, HM_K = 64, HM_LD = HM_K + 8, HM_THREADS = 128;

__device__ __forceinline__ void hm_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

__global__ void __launch_bounds__(HM_THREADS)
head_linear_mma_kernel(const bf16* __restrict__ in, long long ld_in, int in_off, int in_stride, const bf16* __restrict__ w,
                       bf16* __restrict__ out, long long ld_out, int out_off, int out_stride, int n, int n_in, int n_out,
                       const bf16* __restrict__ gate, long long ld_gate) {
  __shared__ __align__(16) bf16 a_s[HM_TILE * HM_LD];
  __shared__ __align__(16) bf16 b_s[HM_TILE * HM_LD];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.z, row0 = blockIdx.x * HM_TILE, col0 = blockIdx.y * HM_TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wr = (warp >> 1) * 32, wc = (warp & 1) * 32;
  const bf16* a_g = in + in_off + (long long)h * in_stride;
  const bf16* b_g = w + (long long)h * n_out * n_in;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  for (int k0 = 0; k0 < n_in; k0 += HM_K) {
    __syncthreads();                                   // the tiles of the chunk before have been read
    for (int e = tid; e < HM_TILE * (HM_K / 8); e += HM_THREADS) {
      const int r = e / (HM_K / 8), c = (e % (HM_K / 8)) * 8;
      const bool col_ok = k0 + c < n_in;
      const bool a_ok = col_ok && row0 + r < n, b_ok = col_ok && col0 + r < n_out;
      hm_cp_async16(a_s + r * HM_LD + c, a_ok ? a_g + (long long)(row0 + r) * ld_in + k0 + c : a_g, a_ok);
      hm_cp_async16(b_s + r * HM_LD + c, b_ok ? b_g + (long long)(col0 + r) * n_in + k0 + c : b_g, b_ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HM_K; kk += 16) {
      uint32_t a0[4], a1[4], b0[4], b1[4];
      load_a(a0, a_s, HM_LD, wr, kk, lane);
      load_a(a1, a_s, HM_LD, wr + 16, kk, lane);
      load_b_pair(b0, b_s, HM_LD, wc, kk, lane);
      load_b_pair(b1, b_s, HM_LD, wc + 16, kk, lane);
      mma_bf16(acc[0][0], a0, b0[0], b0[1]); mma_bf16(acc[0][1], a0, b0[2], b0[3]);
      mma_bf16(acc[0][2], a0, b1[0], b1[1]); mma_bf16(acc[0][3], a0, b1[2], b1[3]);
      mma_bf16(acc[1][0], a1, b0[0], b0[1]); mma_bf16(acc[1][1], a1, b0[2], b0[3]);
      mma_bf16(acc[1][2], a1, b1[0], b1[1]); mma_bf16(acc[1][3], a1, b1[2], b1[3]);
    }
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row0 + wr + mt * 16 + (lane >> 2) + 8 * half;
      if (row >= n) continue;
      float gv = 1.f;
      if (gate != nullptr) gv = 1.f / (1.f + expf(-__bfloat162float(gate[(long long)row * ld_gate + h])));
      bf16* dst = out + (long long)row * ld_out + out_off + (long long)h * out_stride;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = col0 + wc + nt * 8 + 2 * (lane & 3) + e;
          if (col < n_out) dst[col] = __float2bfloat16_rn(acc[mt][nt][2 * half + e] * gv);
        }
    }
}

bool head_linear_mma_takes(const void* in, long long ld_in, int in_off, int in_stride, const void* w, int n_in) {
  return n_in % 8 == 0 && ld_in % 8 == 0 && in_off % 8 == 0 && in_stride % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)w % 16 == 0;
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
  if (dtype == HFEE_BF16 && head_linear_mma_takes(in, ld_in, in_off, in_stride, w, n_in)) {
    hfee_launch(head_linear_mma_kernel, dim3((unsigned)((n + HM_TILE - 1) / HM_TILE), (unsigned)((n_out + HM_TILE - 1) / HM_TILE), (unsigned)heads),
                dim3(HM_THREADS), 0, stream, (const bf16*)in, ld_in, in_off, in_stride, (const bf16*)w, (bf16*)out, ld_out, out_off,
                out_stride, n, n_in, n_out, (const bf16*)gate, ld_gate);
    return hfee_check_launch("head_linear_mma");
  }
  if (dtype == HFEE_BF16)
    return launch_head_linear<__nv_bfloat16>(in, ld_in, in_off, in_stride, w, out, ld_out, out_off, out_stride, n, heads, n_in, n_out, gate, ld_gate, stream);
  return hfee_fail(HFEE_ERR_ARG, "head_linear: unknown dtype %d", dtype);
}
