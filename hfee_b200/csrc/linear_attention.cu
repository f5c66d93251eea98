// Linear attention with a scalar decay per head and a float32 state per (request, head):
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T          S: [dim][vdim], zero for a fresh request
//   o_t = S_t^T q_t
//
// q, k and v are slices of one projection buffer (type T) and pass through an activation
// (none or SiLU) on the way in; the decay, the state, every product and o are float32.
//
// hfee_linear_attention walks a request's tokens one after the other: the kernel of decode steps
// and of the true 32-bit path, and the definition the chunked kernel is tested against.  A thread
// keeps LA_ROWS rows of one state column in registers; a block covers LA_COLS columns and all
// rows (blockDim.y = ceil(dim / LA_ROWS) row groups, whose partial outputs meet in shared memory);
// tokens are staged LA_STAGE at a time.
//
// hfee_linear_attention_chunked is the prompt kernel: runs of LC_T tokens.  With
// a_t = decay^(t+1) (t counts inside the run) a run computes
//
//   o_t = a_t * S_in^T q_t + sum_{s <= t} decay^(t-s) (q_t . k_s) v_s
//   S_out = decay^n S_in + sum_s decay^(n-1-s) k_s v_s^T
//
// which is the recurrence written out.  Three passes so that the runs of a long prompt work in
// parallel: (1) every run's own sum  sum_s decay^(n-1-s) k_s v_s^T, (2) per (request, head,
// column tile) the states in front of every run, in order, and the request's new state, (3)
// every run's outputs from the state in front of it.  All in float32 on the CUDA cores.
#include "common.cuh"

namespace {

constexpr int LA_ROWS = 64;
constexpr int LA_COLS = 64;
constexpr int LA_STAGE = 16;
constexpr int LA_MAX_DIM = 256;

enum Activation { ACT_NONE = 0, ACT_SILU = 1 };

template <int ACT> __device__ __forceinline__ float activate(float z) {
  if constexpr (ACT == ACT_SILU) return z / (1.f + expf(-z));
  return z;
}

template <typename T, int ACT>
__global__ void __launch_bounds__(LA_COLS * (LA_MAX_DIM / LA_ROWS))
linear_attention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                        const float* __restrict__ decay, float* __restrict__ state,
                        const int* __restrict__ cu_tokens, const int* __restrict__ slots, float* __restrict__ out,
                        long long ld_o, int heads, int dim, int vdim, int write_state) {
  extern __shared__ __align__(16) float smem[];
  const int head = blockIdx.x, req = blockIdx.y;
  const int groups = blockDim.y, dim_pad = groups * LA_ROWS;
  const int j = threadIdx.x, g = threadIdx.y;
  const int col = blockIdx.z * LA_COLS + j;
  const int tid = g * LA_COLS + j, threads = LA_COLS * groups;
  float* qs = smem;                                  // [LA_STAGE][dim_pad]
  float* ks = qs + LA_STAGE * dim_pad;               // [LA_STAGE][dim_pad]
  float* vs = ks + LA_STAGE * dim_pad;               // [LA_STAGE][LA_COLS]
  float* part = vs + LA_STAGE * LA_COLS;             // [LA_STAGE][groups][LA_COLS]
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req];
  const float lam = decay[head];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;

  float* S_g = state + (((long long)slot * heads + head) * dim) * vdim;
  float S[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int row = g * LA_ROWS + i;
    S[i] = (row < dim && col < vdim) ? S_g[(long long)row * vdim + col] : 0.f;
  }
  for (int t0 = 0; t0 < count; t0 += LA_STAGE) {
    const int nt = min(LA_STAGE, count - t0);
    __syncthreads();                                 // the stage before is used up
    for (int e = tid; e < nt * dim_pad; e += threads) {
      const int t = e / dim_pad, d = e % dim_pad;
      const long long at = (long long)(begin + t0 + t) * ld + (long long)head * dim + d;
      qs[e] = d < dim ? activate<ACT>(to_f32<T>(q[at])) : 0.f;
      ks[e] = d < dim ? activate<ACT>(to_f32<T>(k[at])) : 0.f;
    }
    for (int e = tid; e < nt * LA_COLS; e += threads) {
      const int t = e / LA_COLS, c = blockIdx.z * LA_COLS + e % LA_COLS;
      vs[e] = c < vdim ? activate<ACT>(to_f32<T>(v[(long long)(begin + t0 + t) * ld + (long long)head * vdim + c])) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float vv = vs[t * LA_COLS + j];
      const float4* k4 = reinterpret_cast<const float4*>(ks + t * dim_pad + g * LA_ROWS);
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * dim_pad + g * LA_ROWS);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < LA_ROWS / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        S[4 * i + 0] = fmaf(lam, S[4 * i + 0], kk.x * vv);  acc = fmaf(S[4 * i + 0], qq.x, acc);
        S[4 * i + 1] = fmaf(lam, S[4 * i + 1], kk.y * vv);  acc = fmaf(S[4 * i + 1], qq.y, acc);
        S[4 * i + 2] = fmaf(lam, S[4 * i + 2], kk.z * vv);  acc = fmaf(S[4 * i + 2], qq.z, acc);
        S[4 * i + 3] = fmaf(lam, S[4 * i + 3], kk.w * vv);  acc = fmaf(S[4 * i + 3], qq.w, acc);
      }
      part[(t * groups + g) * LA_COLS + j] = acc;
    }
    __syncthreads();
    for (int e = tid; e < nt * LA_COLS; e += threads) {
      const int t = e / LA_COLS, jj = e % LA_COLS, c = blockIdx.z * LA_COLS + jj;
      float sum = 0.f;
      for (int gg = 0; gg < groups; ++gg) sum += part[(t * groups + gg) * LA_COLS + jj];
      if (c < vdim) out[(long long)(begin + t0 + t) * ld_o + (long long)head * vdim + c] = sum;
    }
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < LA_ROWS; ++i) {
      const int row = g * LA_ROWS + i;
      if (row < dim && col < vdim) S_g[(long long)row * vdim + col] = S[i];
    }
  }
}

// ------------------------------------------------------------------------------------------ chunked
constexpr int LC_T = 32;          // tokens of a run
constexpr int LC_COLS = 64;       // value columns of a block
constexpr int LC_THREADS = 256;

// The runs of all requests are numbered in batch order: request r's runs start at the sum over earlier
// requests of ceil(count / LC_T).  A block finds (request, run within the request) for its number.
__device__ __forceinline__ int runs_of(int count) { return (count + LC_T - 1) / LC_T; }

__device__ __forceinline__ bool find_run(const int* __restrict__ cu_tokens, int requests, int number, int* req, int* run) {
  int base = 0;
  for (int r = 0; r < requests; ++r) {
    const int c = runs_of(cu_tokens[r + 1] - cu_tokens[r]);
    if (number < base + c) { *req = r; *run = number - base; return true; }
    base += c;
  }
  return false;
}

// (1) sums[run number][head] = sum_s decay^(n-1-s) k_s v_s^T for the run's n tokens, [dim][vdim] each
template <typename T, int ACT>
__global__ void __launch_bounds__(LC_THREADS)
la_chunk_sums_kernel(const T* __restrict__ k, const T* __restrict__ v, long long ld, const float* __restrict__ decay,
                     const int* __restrict__ cu_tokens, float* __restrict__ sums, int requests, int heads, int dim,
                     int vdim) {
  extern __shared__ __align__(16) float smem[];
  const int head = blockIdx.x;
  const int c0 = blockIdx.z * LC_COLS;
  int req = 0, run = 0;
  const bool mine = find_run(cu_tokens, requests, blockIdx.y, &req, &run);
  pdl_wait();
  pdl_launch_dependents();
  if (!mine) return;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int t0 = run * LC_T, n = min(LC_T, count - t0);
  const float lam = decay[head];
  float* ks = smem;                 // [LC_T][dim]   k_s * decay^(n-1-s)
  float* vs = ks + LC_T * dim;      // [LC_T][LC_COLS]
  for (int e = threadIdx.x; e < n * dim; e += LC_THREADS) {
    const int s = e / dim, d = e % dim;
    const float kv = activate<ACT>(to_f32<T>(k[(long long)(begin + t0 + s) * ld + (long long)head * dim + d]));
    ks[e] = kv * powf(lam, (float)(n - 1 - s));
  }
  for (int e = threadIdx.x; e < n * LC_COLS; e += LC_THREADS) {
    const int s = e / LC_COLS, c = c0 + e % LC_COLS;
    vs[e] = c < vdim ? activate<ACT>(to_f32<T>(v[(long long)(begin + t0 + s) * ld + (long long)head * vdim + c])) : 0.f;
  }
  __syncthreads();
  float* A = sums + (((long long)blockIdx.y * heads + head) * dim) * vdim;
  for (int e = threadIdx.x; e < dim * LC_COLS; e += LC_THREADS) {
    const int d = e / LC_COLS, jj = e % LC_COLS;
    float acc = 0.f;
    for (int s = 0; s < n; ++s) acc = fmaf(ks[s * dim + d], vs[s * LC_COLS + jj], acc);
    if (c0 + jj < vdim) A[(long long)d * vdim + c0 + jj] = acc;
  }
}

// (2) in place: sums[run] becomes the state in front of run `run`; the request's state becomes the one
// behind its last run.  One thread per state element walks the runs in order.
__global__ void la_chunk_scan_kernel(const float* __restrict__ decay, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ slots, float* __restrict__ sums, float* __restrict__ state,
                                     int heads, int dim, int vdim, int write_state) {
  const int head = blockIdx.x, req = blockIdx.y;
  const int count = cu_tokens[req + 1] - cu_tokens[req];
  const int slot = slots[req];
  int first_run = 0;
  for (int r = 0; r < req; ++r) first_run += runs_of(cu_tokens[r + 1] - cu_tokens[r]);
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  const float lam = decay[head];
  const int runs = runs_of(count);
  const long long per = (long long)dim * vdim;
  float* S_g = state + ((long long)slot * heads + head) * per;
  for (long long e = (long long)blockIdx.z * blockDim.x + threadIdx.x; e < per; e += (long long)gridDim.z * blockDim.x) {
    float S = S_g[e];
    for (int run = 0; run < runs; ++run) {
      const int n = min(LC_T, count - run * LC_T);
      float* A = sums + ((long long)(first_run + run) * heads + head) * per + e;
      const float own = *A;
      *A = S;
      S = fmaf(powf(lam, (float)n), S, own);
    }
    if (write_state) S_g[e] = S;
  }
}

// (3) o_t = decay^(t+1) S_in^T q_t + sum_{s <= t} decay^(t-s) (q_t . k_s) v_s
template <typename T, int ACT>
__global__ void __launch_bounds__(LC_THREADS)
la_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                    const float* __restrict__ decay, const int* __restrict__ cu_tokens, const float* __restrict__ sums,
                    float* __restrict__ out, long long ld_o, int requests, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  const int head = blockIdx.x;
  const int c0 = blockIdx.z * LC_COLS;
  int req = 0, run = 0;
  const bool mine = find_run(cu_tokens, requests, blockIdx.y, &req, &run);
  pdl_wait();
  pdl_launch_dependents();
  if (!mine) return;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int t0 = run * LC_T, n = min(LC_T, count - t0);
  const float lam = decay[head];
  float* qs = smem;                    // [LC_T][dim + 1]
  float* ks = qs + LC_T * (dim + 1);   // [LC_T][dim + 1]
  float* vs = ks + LC_T * (dim + 1);   // [LC_T][LC_COLS]
  float* ps = vs + LC_T * LC_COLS;     // [LC_T][LC_T]   decay^(t-s) (q_t . k_s), 0 for s > t
  const int ldq = dim + 1;
  for (int e = threadIdx.x; e < n * dim; e += LC_THREADS) {
    const int s = e / dim, d = e % dim;
    const long long at = (long long)(begin + t0 + s) * ld + (long long)head * dim + d;
    qs[s * ldq + d] = activate<ACT>(to_f32<T>(q[at]));
    ks[s * ldq + d] = activate<ACT>(to_f32<T>(k[at]));
  }
  for (int e = threadIdx.x; e < n * LC_COLS; e += LC_THREADS) {
    const int s = e / LC_COLS, c = c0 + e % LC_COLS;
    vs[e] = c < vdim ? activate<ACT>(to_f32<T>(v[(long long)(begin + t0 + s) * ld + (long long)head * vdim + c])) : 0.f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n * LC_T; e += LC_THREADS) {
    const int t = e / LC_T, s = e % LC_T;
    float acc = 0.f;
    if (s <= t) {
      for (int d = 0; d < dim; ++d) acc = fmaf(qs[t * ldq + d], ks[s * ldq + d], acc);
      acc *= powf(lam, (float)(t - s));
    }
    ps[e] = acc;
  }
  __syncthreads();
  const float* S_in = sums + (((long long)blockIdx.y * heads + head) * dim) * vdim;
  for (int e = threadIdx.x; e < n * LC_COLS; e += LC_THREADS) {
    const int t = e / LC_COLS, jj = e % LC_COLS, c = c0 + jj;
    if (c >= vdim) continue;
    float inter = 0.f;
    for (int d = 0; d < dim; ++d) inter = fmaf(qs[t * ldq + d], S_in[(long long)d * vdim + c], inter);
    float intra = 0.f;
    for (int s = 0; s <= t; ++s) intra = fmaf(ps[t * LC_T + s], vs[s * LC_COLS + jj], intra);
    out[(long long)(begin + t0 + t) * ld_o + (long long)head * vdim + c] = fmaf(powf(lam, (float)(t + 1)), inter, intra);
  }
}

template <typename T>
int launch_recurrent(const void* q, const void* k, const void* v, long long ld, const float* decay, float* state,
                     const int* cu_tokens, const int* slots, float* out, long long ld_o, int requests, int heads, int dim,
                     int vdim, int activation, int write_state, cudaStream_t stream) {
  const int groups = (dim + LA_ROWS - 1) / LA_ROWS, dim_pad = groups * LA_ROWS;
  const size_t smem = sizeof(float) * (size_t)LA_STAGE * (2 * dim_pad + LA_COLS + groups * LA_COLS);
  const dim3 grid(heads, requests, (vdim + LA_COLS - 1) / LA_COLS), block(LA_COLS, groups);
  auto go = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hfee_launch(kernel, grid, block, smem, stream, (const T*)q, (const T*)k, (const T*)v, ld, decay, state, cu_tokens,
                slots, out, ld_o, heads, dim, vdim, write_state);
  };
  if (activation == ACT_SILU) go(linear_attention_kernel<T, ACT_SILU>);
  else go(linear_attention_kernel<T, ACT_NONE>);
  return hfee_check_launch("linear_attention");
}

template <typename T>
int launch_chunked(const void* q, const void* k, const void* v, long long ld, const float* decay, float* state,
                   const int* cu_tokens, const int* slots, float* out, long long ld_o, float* sums, int requests,
                   int tokens, int heads, int dim, int vdim, int activation, int write_state, cudaStream_t stream) {
  const unsigned tiles = (unsigned)((vdim + LC_COLS - 1) / LC_COLS);
  const dim3 grid(heads, (unsigned)(tokens / LC_T + requests), tiles);     // at least as many as there are runs
  const size_t smem1 = sizeof(float) * (size_t)LC_T * (dim + LC_COLS);
  const size_t smem3 = sizeof(float) * (size_t)LC_T * (2 * (dim + 1) + LC_COLS + LC_T);
  auto go = [&](auto sums_kernel, auto out_kernel) {
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (smem3 > 48 * 1024) cudaFuncSetAttribute(out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    hfee_launch(sums_kernel, grid, dim3(LC_THREADS), smem1, stream, (const T*)k, (const T*)v, ld, decay, cu_tokens, sums,
                requests, heads, dim, vdim);
    const long long per = (long long)dim * vdim;
    const unsigned z = (unsigned)((per + 255) / 256 < 64 ? (per + 255) / 256 : 64);
    hfee_launch(la_chunk_scan_kernel, dim3(heads, requests, z), dim3(256), 0, stream, decay, cu_tokens, slots, sums, state,
                heads, dim, vdim, write_state);
    hfee_launch(out_kernel, grid, dim3(LC_THREADS), smem3, stream, (const T*)q, (const T*)k, (const T*)v, ld, decay,
                cu_tokens, (const float*)sums, out, ld_o, requests, heads, dim, vdim);
  };
  if (activation == ACT_SILU) go(la_chunk_sums_kernel<T, ACT_SILU>, la_chunk_out_kernel<T, ACT_SILU>);
  else go(la_chunk_sums_kernel<T, ACT_NONE>, la_chunk_out_kernel<T, ACT_NONE>);
  return hfee_check_launch("linear_attention_chunked");
}

int check_sizes(const char* what, int requests, int heads, int dim, int vdim, long long ld, long long ld_o, int activation) {
  HFEE_REQUIRE(requests > 0 && heads > 0 && dim > 0 && vdim > 0, "%s: bad sizes", what);
  HFEE_REQUIRE(dim <= LA_MAX_DIM, "%s: key size %d is above %d", what, dim, LA_MAX_DIM);
  HFEE_REQUIRE(ld >= (long long)heads * (dim > vdim ? dim : vdim) && ld_o >= (long long)heads * vdim,
               "%s: a leading dimension is too small", what);
  HFEE_REQUIRE(activation == ACT_NONE || activation == ACT_SILU, "%s: unknown activation %d", what, activation);
  return HFEE_OK;
}

}  // namespace

HFEE_API int hfee_linear_attention(const void* q, const void* k, const void* v, long long ld, int dtype,
                                   const float* decay, float* state, const int* cu_tokens, const int* slots, float* out,
                                   long long ld_o, int requests, int heads, int dim, int vdim, int activation,
                                   int write_state, cudaStream_t stream) {
  if (requests == 0) return HFEE_OK;
  if (int e = check_sizes("linear_attention", requests, heads, dim, vdim, ld, ld_o, activation)) return e;
  if (dtype == HFEE_F32)
    return launch_recurrent<float>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, requests, heads, dim, vdim, activation, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_recurrent<__nv_bfloat16>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, requests, heads, dim, vdim, activation, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "linear_attention: unknown dtype %d", dtype);
}

// floats of workspace the chunked kernel needs for a step of `tokens` tokens in `requests` requests
HFEE_API long long hfee_linear_attention_chunked_workspace(int requests, int tokens, int heads, int dim, int vdim) {
  return (long long)(tokens / LC_T + requests) * heads * dim * vdim;
}

HFEE_API int hfee_linear_attention_chunked(const void* q, const void* k, const void* v, long long ld, int dtype,
                                           const float* decay, float* state, const int* cu_tokens, const int* slots,
                                           float* out, long long ld_o, float* workspace, long long workspace_floats,
                                           int requests, int tokens, int heads, int dim, int vdim, int activation,
                                           int write_state, cudaStream_t stream) {
  if (requests == 0 || tokens == 0) return HFEE_OK;
  if (int e = check_sizes("linear_attention_chunked", requests, heads, dim, vdim, ld, ld_o, activation)) return e;
  HFEE_REQUIRE(workspace != nullptr && workspace_floats >= hfee_linear_attention_chunked_workspace(requests, tokens, heads, dim, vdim),
               "linear_attention_chunked: the workspace is too small");
  if (dtype == HFEE_F32)
    return launch_chunked<float>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, workspace, requests, tokens, heads, dim, vdim, activation, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_chunked<__nv_bfloat16>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, workspace, requests, tokens, heads, dim, vdim, activation, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "linear_attention_chunked: unknown dtype %d", dtype);
}
