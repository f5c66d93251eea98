// The gated delta rule on a matrix state per head, and the short convolution with activation in front of it.
//
//   hfee_conv_act     y[t, c] = act(sum_j w[c, j] * x[t - taps + 1 + j, c]) per request, inputs in front of the step's
//                     tokens taken from the request's state (its last taps - 1 inputs, zeros for a fresh request),
//                     which is renewed.  x is a slice of a projection (any row stride, either dtype); arithmetic and
//                     state are float32.
//   hfee_delta_rule   per request and head, with S [dim, vdim] float32 carried from step to step:
//                         S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//                     q and k are first made unit vectors (x / sqrt(sum x^2 + 1e-6); q also times dim^-1/2),
//                     beta_t = sigmoid(b_t), g_t = exp(-exp(A_log) * softplus(a_t + dt_bias)), all float32.
//                     Columns of S evolve independently: S[:, j] <- g S[:, j] + k * beta (v_j - g S[:, j].k), so a
//                     block owns DR_COLS columns of one (request, head), DR_LANES lanes share a column (each keeps
//                     dim / DR_LANES of its entries in registers), and the tokens of the step are walked in order:
//                     the result does not depend on how a prompt was cut.  Tiles of DR_TILE tokens are staged in
//                     shared memory (normalised there) between two barriers.
#include "common.cuh"

namespace {

constexpr int CA_MAX_TAPS = 8;
constexpr int CA_TOKENS = 16;
constexpr int CA_THREADS = 128;
constexpr int CA_OUT = 1, CA_STATE = 2;
constexpr int ACT_NONE = 0, ACT_SILU = 1;

template <typename T>
__global__ void __launch_bounds__(CA_THREADS)
conv_act_kernel(const T* __restrict__ x, long long ld_x, const float* __restrict__ w, float* __restrict__ state,
                const int* __restrict__ cu_tokens, const int* __restrict__ slots, T* __restrict__ out, long long ld_out,
                int width, int taps, int act, int mode) {
  const int req = blockIdx.y;
  const int c = blockIdx.z * CA_THREADS + threadIdx.x;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;     // host-written batch layout
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0 || c >= width) return;
  const int hist = taps - 1;
  const int first = (mode == CA_STATE) ? ((count - 1) / CA_TOKENS) * CA_TOKENS : blockIdx.x * CA_TOKENS;
  if (first >= count) return;
  const int last = min(count, first + CA_TOKENS);
  float* st = state + (long long)slot * hist * width + c;                    // st[s * width]: input at index s - hist
  const T* xc = x + (long long)begin * ld_x + c;
  float wv[CA_MAX_TAPS], win[CA_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CA_MAX_TAPS; ++j) {
    wv[j] = j < taps ? w[(long long)c * taps + j] : 0.f;
    win[j] = 0.f;
    if (j < hist) {
      const int s = first - hist + j;
      win[j] = s >= 0 ? to_f32<T>(xc[(long long)s * ld_x]) : st[(long long)(hist + s) * width];
    }
  }
  if (mode & CA_OUT) {
    for (int t = first; t < last; ++t) {
      const float xv = to_f32<T>(xc[(long long)t * ld_x]);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < CA_MAX_TAPS; ++j) {
        const float in = (j == hist) ? xv : win[j];
        if (j < taps) acc = fmaf(wv[j], in, acc);
      }
      if (act == ACT_SILU) acc = acc / (1.f + expf(-acc));
      out[(long long)(begin + t) * ld_out + c] = from_f32<T>(acc);
#pragma unroll
      for (int j = 0; j + 1 < CA_MAX_TAPS; ++j) win[j] = (j + 1 == hist) ? xv : win[j + 1];
    }
  }
  if ((mode & CA_STATE) && last == count) {
    // new st[s] = input at index count - hist + s; a negative index lies in the old state, at a higher
    // place than the one being written, so ascending order reads before it overwrites
    for (int s = 0; s < hist; ++s) {
      const int idx = count - hist + s;
      st[(long long)s * width] = idx >= 0 ? to_f32<T>(xc[(long long)idx * ld_x]) : st[(long long)(hist + idx) * width];
    }
  }
}

template <typename T>
int launch_conv_act(const void* x, long long ld_x, const float* w, float* state, const int* cu_tokens, const int* slots,
                    void* out, long long ld_out, int requests, int max_new, int width, int taps, int act, int write_state,
                    cudaStream_t stream) {
  const unsigned runs = (unsigned)((max_new + CA_TOKENS - 1) / CA_TOKENS);
  const unsigned cz = (unsigned)((width + CA_THREADS - 1) / CA_THREADS);
  const bool together = write_state && runs == 1 && taps > 1;
  hfee_launch(conv_act_kernel<T>, dim3(runs, requests, cz), dim3(CA_THREADS), 0, stream, (const T*)x, ld_x, w, state, cu_tokens,
              slots, (T*)out, ld_out, width, taps, act, together ? (CA_OUT | CA_STATE) : CA_OUT);
  if (write_state && !together && taps > 1)
    hfee_launch(conv_act_kernel<T>, dim3(1, requests, cz), dim3(CA_THREADS), 0, stream, (const T*)x, ld_x, w, state, cu_tokens,
                slots, (T*)out, ld_out, width, taps, act, CA_STATE);
  return hfee_check_launch("conv_act");
}

// ---------------------------------------------------------------------------------------------------------------
constexpr int DR_LANES = 8;                  // lanes that share a column of the state
constexpr int DR_THREADS = 128;
constexpr int DR_COLS = DR_THREADS / DR_LANES;
constexpr int DR_TILE = 16;                  // tokens staged at once
constexpr int DR_MAX_DIM = 256;

__device__ __forceinline__ float group_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaArgs {
  long long ld_qkv, ld_ba, ld_out;
  int q_off, k_off, v_off;         // columns of head 0 in a row of the q/k/v buffer
  int b_off, a_off;                // columns of head 0's write strength and decay inputs
  int heads, qk_heads, dim, vdim;
  int write_state;
};

// R: state entries per lane (dim <= DR_LANES * R)
template <typename T, int R>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const T* __restrict__ qkv, const T* __restrict__ ba, const float* __restrict__ a_log,
                  const float* __restrict__ dt_bias, float* __restrict__ state, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, float* __restrict__ out, DeltaArgs p) {
  constexpr int DP = DR_LANES * R;           // padded key size
  extern __shared__ float smem[];
  float* q_s = smem;                         // [DR_TILE][DP]
  float* k_s = q_s + DR_TILE * DP;           // [DR_TILE][DP]
  __shared__ float v_s[DR_TILE][DR_COLS], o_s[DR_TILE][DR_COLS], beta_s[DR_TILE], g_s[DR_TILE];
  const int req = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * DR_COLS;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = tid / DR_LANES, lg = tid % DR_LANES;
  const int col = col0 + grp;
  const int kh = h / (p.heads / p.qk_heads);
  const int dim = p.dim, vdim = p.vdim;
  float* sp = state + (((long long)slot * p.heads + h) * dim) * vdim + col;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lg + DR_LANES * r;
    S[r] = (i < dim && col < vdim) ? sp[(long long)i * vdim] : 0.f;
  }
  const float rate = expf(a_log[h]), bias = dt_bias[h];
  const float q_scale = 1.0f / sqrtf((float)dim);

  for (int tile0 = 0; tile0 < count; tile0 += DR_TILE) {
    const int tt = min(DR_TILE, count - tile0);
    const long long tok0 = begin + tile0;
    for (int e = tid; e < tt * DP; e += DR_THREADS) {
      const int t = e / DP, d = e - t * DP;
      const T* row = qkv + (tok0 + t) * p.ld_qkv + (long long)kh * dim + d;
      q_s[e] = d < dim ? to_f32<T>(row[p.q_off]) : 0.f;
      k_s[e] = d < dim ? to_f32<T>(row[p.k_off]) : 0.f;
    }
    for (int e = tid; e < tt * DR_COLS; e += DR_THREADS) {
      const int t = e / DR_COLS, c = e - t * DR_COLS;
      v_s[t][c] = col0 + c < vdim ? to_f32<T>(qkv[(tok0 + t) * p.ld_qkv + p.v_off + (long long)h * vdim + col0 + c]) : 0.f;
    }
    if (tid < tt) {
      const T* row = ba + (tok0 + tid) * p.ld_ba;
      beta_s[tid] = 1.f / (1.f + expf(-to_f32<T>(row[p.b_off + h])));
      g_s[tid] = expf(-rate * softplus_f32(to_f32<T>(row[p.a_off + h]) + bias));
    }
    __syncthreads();
    for (int vid = warp; vid < 2 * tt; vid += DR_THREADS / 32) {
      float* vec = vid < tt ? q_s + vid * DP : k_s + (vid - tt) * DP;
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(vec[d], vec[d], ss);
      const float scale = (vid < tt ? q_scale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
      for (int d = lane; d < dim; d += 32) vec[d] *= scale;
    }
    __syncthreads();
    for (int t = 0; t < tt; ++t) {
      const float* kt = k_s + t * DP + lg;
      const float* qt = q_s + t * DP + lg;
      float kk[R];
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        kk[r] = kt[DR_LANES * r];
        s = fmaf(S[r], kk[r], s);
      }
      s = group_sum(s);
      const float g = g_s[t];
      const float u = beta_s[t] * (v_s[t][grp] - g * s);
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        S[r] = fmaf(kk[r], u, g * S[r]);
        o = fmaf(S[r], qt[DR_LANES * r], o);
      }
      o = group_sum(o);
      if (lg == 0) o_s[t][grp] = o;
    }
    __syncthreads();
    for (int e = tid; e < tt * DR_COLS; e += DR_THREADS) {
      const int t = e / DR_COLS, c = e - t * DR_COLS;
      if (col0 + c < vdim) out[(tok0 + t) * p.ld_out + (long long)h * vdim + col0 + c] = o_s[t][c];
    }
  }
  if (p.write_state) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = lg + DR_LANES * r;
      if (i < dim && col < vdim) sp[(long long)i * vdim] = S[r];
    }
  }
}

template <typename T, int R>
int launch_delta_r(const void* qkv, const void* ba, const float* a_log, const float* dt_bias, float* state,
                   const int* cu_tokens, const int* slots, float* out, const DeltaArgs& p, int requests, cudaStream_t stream) {
  const size_t smem = (size_t)2 * DR_TILE * DR_LANES * R * sizeof(float);
  hfee_launch(delta_rule_kernel<T, R>, dim3((unsigned)((p.vdim + DR_COLS - 1) / DR_COLS), (unsigned)p.heads, (unsigned)requests),
              dim3(DR_THREADS), smem, stream, (const T*)qkv, (const T*)ba, a_log, dt_bias, state, cu_tokens, slots, out, p);
  return hfee_check_launch("delta_rule");
}

template <typename T>
int launch_delta(const void* qkv, const void* ba, const float* a_log, const float* dt_bias, float* state,
                 const int* cu_tokens, const int* slots, float* out, const DeltaArgs& p, int requests, cudaStream_t stream) {
  const int r = (p.dim + DR_LANES - 1) / DR_LANES;
  if (r <= 1) return launch_delta_r<T, 1>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 2) return launch_delta_r<T, 2>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 4) return launch_delta_r<T, 4>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 8) return launch_delta_r<T, 8>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (r <= 16) return launch_delta_r<T, 16>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  return launch_delta_r<T, 32>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
}

}  // namespace

// Launches one kernel, or two when a portion is longer than one run of tokens and the state is written.
HFEE_API int hfee_conv_act_launches(int max_new, int taps, int write_state) {
  return (write_state && taps > 1 && max_new > CA_TOKENS) ? 2 : 1;
}

// act: 0 none, 1 SiLU.  state: [slots, taps - 1, width] float32.
HFEE_API int hfee_conv_act(const void* x, long long ld_x, int dtype, const float* w, float* state, const int* cu_tokens,
                           const int* slots, void* out, long long ld_out, int requests, int max_new, int width, int taps,
                           int act, int write_state, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(requests > 0 && max_new > 0 && width > 0, "conv_act: bad sizes");
  HFEE_REQUIRE(taps >= 1 && taps <= CA_MAX_TAPS, "conv_act: taps %d is outside 1..%d", taps, CA_MAX_TAPS);
  HFEE_REQUIRE(ld_x >= width && ld_out >= width, "conv_act: a row stride is too small");
  HFEE_REQUIRE(act == ACT_NONE || act == ACT_SILU, "conv_act: unknown activation %d", act);
  if (dtype == HFEE_F32)
    return launch_conv_act<float>(x, ld_x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_conv_act<__nv_bfloat16>(x, ld_x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, act, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "conv_act: unknown dtype %d", dtype);
}

// qkv rows: head g's query at q_off + g * dim, its key at k_off + g * dim (g < qk_heads; head h of `heads` uses
// g = h / (heads / qk_heads)), head h's value at v_off + h * vdim.  ba rows: b_off + h and a_off + h.
// state: [slots, heads, dim, vdim] float32.  out: float32 [n, heads * vdim].
HFEE_API int hfee_delta_rule(const void* qkv, long long ld_qkv, int q_off, int k_off, int v_off, const void* ba,
                             long long ld_ba, int b_off, int a_off, int dtype, const float* a_log, const float* dt_bias,
                             float* state, const int* cu_tokens, const int* slots, float* out, long long ld_out,
                             int requests, int heads, int qk_heads, int dim, int vdim, int write_state,
                             cudaStream_t stream) {
  if (requests == 0) return HFEE_OK;
  HFEE_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0, "delta_rule: heads %d must be a multiple of %d", heads, qk_heads);
  HFEE_REQUIRE(dim > 0 && dim <= DR_MAX_DIM && vdim > 0, "delta_rule: key size %d is outside 1..%d", dim, DR_MAX_DIM);
  DeltaArgs p{ld_qkv, ld_ba, ld_out, q_off, k_off, v_off, b_off, a_off, heads, qk_heads, dim, vdim, write_state};
  if (dtype == HFEE_F32)
    return launch_delta<float>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  if (dtype == HFEE_BF16)
    return launch_delta<__nv_bfloat16>(qkv, ba, a_log, dt_bias, state, cu_tokens, slots, out, p, requests, stream);
  return hfee_fail(HFEE_ERR_ARG, "delta_rule: unknown dtype %d", dtype);
}
