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
// every run's outputs from the state in front of it.  In float32 on the CUDA cores for float32
// activations and for sizes the tensor-core variant (further down) does not take.
#include "common.cuh"
#include "mma_tiles.cuh"

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

// for activations that are rounded to bfloat16 right away: ex2.approx and a fast division
template <int ACT> __device__ __forceinline__ float activate_fast(float z) {
  if constexpr (ACT == ACT_SILU) return __fdividef(z, 1.f + __expf(-z));
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
template <int RUN> __device__ __forceinline__ int runs_of(int count) { return (count + RUN - 1) / RUN; }

template <int RUN>
__device__ __forceinline__ bool find_run(const int* __restrict__ cu_tokens, int requests, int number, int* req, int* run) {
  int base = 0;
  for (int r = 0; r < requests; ++r) {
    const int c = runs_of<RUN>(cu_tokens[r + 1] - cu_tokens[r]);
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
  const bool mine = find_run<LC_T>(cu_tokens, requests, blockIdx.y, &req, &run);
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
template <int RUN>
__global__ void la_chunk_scan_kernel(const float* __restrict__ decay, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ slots, float* __restrict__ sums, float* __restrict__ state,
                                     int heads, int dim, int vdim, int write_state) {
  const int head = blockIdx.x, req = blockIdx.y;
  const int count = cu_tokens[req + 1] - cu_tokens[req];
  const int slot = slots[req];
  int first_run = 0;
  for (int r = 0; r < req; ++r) first_run += runs_of<RUN>(cu_tokens[r + 1] - cu_tokens[r]);
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0) return;
  const float lam = decay[head];
  const int runs = runs_of<RUN>(count);
  const float lam_full = powf(lam, (float)RUN);
  const float lam_last = powf(lam, (float)(count - (runs - 1) * RUN));      // only the last run can be short
  const long long per = (long long)dim * vdim;
  float* S_g = state + ((long long)slot * heads + head) * per;
  for (long long e = (long long)blockIdx.z * blockDim.x + threadIdx.x; e < per; e += (long long)gridDim.z * blockDim.x) {
    float S = S_g[e];
    float* A0 = sums + ((long long)first_run * heads + head) * per + e;
    const long long stride = (long long)heads * per;
    for (int base = 0; base < runs; base += 8) {          // eight runs' sums are requested before the first is used
      float own[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) own[i] = base + i < runs ? A0[(base + i) * stride] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int run = base + i;
        if (run < runs) {
          A0[run * stride] = S;
          S = fmaf(run == runs - 1 ? lam_last : lam_full, S, own[i]);
        }
      }
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
  const bool mine = find_run<LC_T>(cu_tokens, requests, blockIdx.y, &req, &run);
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


// ------------------------------------------------------------------------------------------ chunked, tensor cores
// The same three passes with runs of LM_T tokens and the products on mma.sync (bfloat16 in, float32 out).
// q, k and v enter as the bfloat16 values of their activations.  Everything else that a product reads is a
// float32 quantity and goes in as the sum of two bfloat16 numbers (the value rounded, and what the rounding
// left), each with a product of its own: the decayed keys k_s decay^(n-1-s), the weights
// decay^(t-s) (q_t . k_s), and the state in front of the run.  Sums are float32.
constexpr int LM_T = 64;
constexpr int LM_COLS = 64;
constexpr int LM_WARPS = 4;
constexpr int LM_PAD = 8;          // bfloat16 per shared-memory row beyond its content: fragment loads meet no bank twice
struct alignas(16) Pack8 { bf16 v[8]; };

// (1) sums[run number][head] = sum_s (k_s decay^(n-1-s)) v_s^T
template <int ACT>
__global__ void __launch_bounds__(LM_WARPS * 32)
la_mma_sums_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, long long ld, const float* __restrict__ decay,
                   const int* __restrict__ cu_tokens, float* __restrict__ sums, int requests, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int head = blockIdx.x, c0 = blockIdx.z * LM_COLS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int req = 0, run = 0;
  const bool mine = find_run<LM_T>(cu_tokens, requests, blockIdx.y, &req, &run);
  pdl_wait();
  pdl_launch_dependents();
  if (!mine) return;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int t0 = run * LM_T, n = min(LM_T, count - t0);
  const float lam = decay[head];
  constexpr int LDT = LM_T + LM_PAD;
  bf16* kt_hi = reinterpret_cast<bf16*>(smem_raw);       // [dim][LDT]  (k_s decay^(n-1-s)) transposed
  bf16* kt_lo = kt_hi + dim * LDT;
  bf16* vt = kt_lo + dim * LDT;                          // [LM_COLS][LDT]
  float* pw = reinterpret_cast<float*>(vt + LM_COLS * LDT);   // decay^i, i = 0..LM_T
  for (int i = threadIdx.x; i <= LM_T; i += LM_WARPS * 32) pw[i] = powf(lam, (float)i);
  __syncthreads();
  // 16-byte loads: a thread takes 8 consecutive dimensions of one token
  const int dv = dim / 8;
  // neighbouring threads take neighbouring tokens, so that the transposed stores meet no bank twice
  // the values' loads first (a fixed number per thread), then the keys' in batches of four: all of a batch's
  // loads are requested before the first is used
  constexpr int V_PER = LM_T * (LM_COLS / 8) / (LM_WARPS * 32);
  Pack8 rv[V_PER];
#pragma unroll
  for (int i = 0; i < V_PER; ++i) {
    const int e = threadIdx.x + i * LM_WARPS * 32, s = e % LM_T, c = c0 + (e / LM_T) * 8;
    rv[i] = Pack8{};
    if (s < n && c < vdim) rv[i] = *reinterpret_cast<const Pack8*>(v + (long long)(begin + t0 + s) * ld + (long long)head * vdim + c);
  }
  for (int e0 = threadIdx.x; e0 < LM_T * dv; e0 += 4 * LM_WARPS * 32) {
    Pack8 raw[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, s = e % LM_T, d = (e / LM_T) * 8;
      raw[b] = Pack8{};
      if (e < LM_T * dv && s < n) raw[b] = *reinterpret_cast<const Pack8*>(k + (long long)(begin + t0 + s) * ld + (long long)head * dim + d);
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, s = e % LM_T, d = (e / LM_T) * 8;
      if (e >= LM_T * dv) break;
      const float w = s < n ? pw[n - 1 - s] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float kb = __bfloat162float(__float2bfloat16_rn(activate_fast<ACT>(__bfloat162float(raw[b].v[i]))));
        split_bf16(kb * w, &kt_hi[(d + i) * LDT + s], &kt_lo[(d + i) * LDT + s]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < V_PER; ++i) {
    const int e = threadIdx.x + i * LM_WARPS * 32, s = e % LM_T, j = (e / LM_T) * 8;
#pragma unroll
    for (int x = 0; x < 8; ++x) vt[(j + x) * LDT + s] = __float2bfloat16_rn(activate_fast<ACT>(__bfloat162float(rv[i].v[x])));
  }
  __syncthreads();
  float* A = sums + (((long long)blockIdx.y * heads + head) * dim) * vdim;
  const int g = lane >> 2, t = lane & 3;
  for (int d0 = warp * 16; d0 < dim; d0 += LM_WARPS * 16) {
    float acc[LM_COLS / 8][4];
#pragma unroll
    for (int nt = 0; nt < LM_COLS / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < LM_T / 16; ++ks) {
      uint32_t ah[4], al[4];
      load_a(ah, kt_hi, LDT, d0, ks * 16, lane);
      load_a(al, kt_lo, LDT, d0, ks * 16, lane);
#pragma unroll
      for (int nt = 0; nt < LM_COLS / 8; nt += 2) {
        uint32_t b[4];
        load_b_pair(b, vt, LDT, nt * 8, ks * 16, lane);
        mma_bf16(acc[nt], ah, b[0], b[1]);
        mma_bf16(acc[nt], al, b[0], b[1]);
        mma_bf16(acc[nt + 1], ah, b[2], b[3]);
        mma_bf16(acc[nt + 1], al, b[2], b[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < LM_COLS / 8; ++nt) {
      const int c = c0 + nt * 8 + 2 * t;
      float* r0 = A + (long long)(d0 + g) * vdim + c;
      float* r1 = A + (long long)(d0 + g + 8) * vdim + c;
      if (c < vdim) { r0[0] = acc[nt][0]; r1[0] = acc[nt][2]; }
      if (c + 1 < vdim) { r0[1] = acc[nt][1]; r1[1] = acc[nt][3]; }
    }
  }
}

// (3) o_t = decay^(t+1) S_in^T q_t + sum_{s <= t} decay^(t-s) (q_t . k_s) v_s; warp w owns rows 16w..16w+15 of the run
template <int ACT>
__global__ void __launch_bounds__(LM_WARPS * 32)
la_mma_out_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, long long ld,
                  const float* __restrict__ decay, const int* __restrict__ cu_tokens, const float* __restrict__ sums,
                  float* __restrict__ out, long long ld_o, int requests, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int head = blockIdx.x, c0 = blockIdx.z * LM_COLS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int req = 0, run = 0;
  const bool mine = find_run<LM_T>(cu_tokens, requests, blockIdx.y, &req, &run);
  pdl_wait();
  pdl_launch_dependents();
  if (!mine) return;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int t0 = run * LM_T, n = min(LM_T, count - t0);
  const float lam = decay[head];
  const int LDD = dim + LM_PAD;
  constexpr int LDT = LM_T + LM_PAD;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);          // [LM_T][LDD]
  bf16* ks_ = qs + LM_T * LDD;                           // [LM_T][LDD]
  bf16* st_hi = ks_ + LM_T * LDD;                        // [LM_COLS][LDD]  the state in front of the run, transposed
  bf16* st_lo = st_hi + LM_COLS * LDD;
  bf16* vt = st_lo + LM_COLS * LDD;                      // [LM_COLS][LDT]
  bf16* p_hi = vt + LM_COLS * LDT;                       // [LM_T][LDT]
  bf16* p_lo = p_hi + LM_T * LDT;
  float* pw = reinterpret_cast<float*>(p_lo + LM_T * LDT);   // decay^i, i = 0..LM_T
  // 16-byte loads: a thread takes 8 consecutive dimensions of one token (4 columns of one state row).  The values'
  // loads go first (a fixed number per thread); queries, keys and the state follow in batches of four whose loads
  // are all requested before the first is used.
  const int dv = dim / 8;
  constexpr int V_PER = LM_T * (LM_COLS / 8) / (LM_WARPS * 32);
  Pack8 rv[V_PER];
#pragma unroll
  for (int i = 0; i < V_PER; ++i) {
    const int e = threadIdx.x + i * LM_WARPS * 32, s = e % LM_T, c = c0 + (e / LM_T) * 8;
    rv[i] = Pack8{};
    if (s < n && c < vdim) rv[i] = *reinterpret_cast<const Pack8*>(v + (long long)(begin + t0 + s) * ld + (long long)head * vdim + c);
  }
  for (int e0 = threadIdx.x; e0 < LM_T * dv; e0 += 4 * LM_WARPS * 32) {
    Pack8 rq[4], rk[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, s = e / dv, d = (e % dv) * 8;
      rq[b] = Pack8{};
      rk[b] = Pack8{};
      if (e < LM_T * dv && s < n) {
        const long long at = (long long)(begin + t0 + s) * ld + (long long)head * dim + d;
        rq[b] = *reinterpret_cast<const Pack8*>(q + at);
        rk[b] = *reinterpret_cast<const Pack8*>(k + at);
      }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, s = e / dv, d = (e % dv) * 8;
      if (e >= LM_T * dv) break;
      Pack8 oq, ok;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        oq.v[i] = __float2bfloat16_rn(activate_fast<ACT>(__bfloat162float(rq[b].v[i])));
        ok.v[i] = __float2bfloat16_rn(activate_fast<ACT>(__bfloat162float(rk[b].v[i])));
      }
      *reinterpret_cast<Pack8*>(qs + s * LDD + d) = oq;
      *reinterpret_cast<Pack8*>(ks_ + s * LDD + d) = ok;
    }
  }
  const float* S_in = sums + (((long long)blockIdx.y * heads + head) * dim) * vdim;
  for (int e0 = threadIdx.x; e0 < dim * (LM_COLS / 4); e0 += 4 * LM_WARPS * 32) {
    float4 x[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, d = e % dim, c = c0 + (e / dim) * 4;   // neighbouring threads: neighbouring state rows
      x[b] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < dim * (LM_COLS / 4) && c < vdim) x[b] = *reinterpret_cast<const float4*>(S_in + (long long)d * vdim + c);
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int e = e0 + b * LM_WARPS * 32, d = e % dim, j = (e / dim) * 4;
      if (e >= dim * (LM_COLS / 4)) break;
      split_bf16(x[b].x, &st_hi[(j + 0) * LDD + d], &st_lo[(j + 0) * LDD + d]);
      split_bf16(x[b].y, &st_hi[(j + 1) * LDD + d], &st_lo[(j + 1) * LDD + d]);
      split_bf16(x[b].z, &st_hi[(j + 2) * LDD + d], &st_lo[(j + 2) * LDD + d]);
      split_bf16(x[b].w, &st_hi[(j + 3) * LDD + d], &st_lo[(j + 3) * LDD + d]);
    }
  }
#pragma unroll
  for (int i = 0; i < V_PER; ++i) {
    const int e = threadIdx.x + i * LM_WARPS * 32, s = e % LM_T, j = (e / LM_T) * 8;
#pragma unroll
    for (int x = 0; x < 8; ++x) vt[(j + x) * LDT + s] = __float2bfloat16_rn(activate_fast<ACT>(__bfloat162float(rv[i].v[x])));
  }
  for (int i = threadIdx.x; i <= LM_T; i += LM_WARPS * 32) pw[i] = powf(lam, (float)i);
  __syncthreads();

  const int g = lane >> 2, t = lane & 3;
  const int r0 = warp * 16;
  if (r0 >= n) return;
  float acc[LM_T / 8][4];
  // weights of the warp's rows: keys in blocks of 8 up to the diagonal
  const int key_tiles = r0 / 8 + 2;
#pragma unroll
  for (int nt = 0; nt < LM_T / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  for (int kk = 0; kk < dim; kk += 16) {
    uint32_t a[4];
    load_a(a, qs, LDD, r0, kk, lane);
#pragma unroll
    for (int nt = 0; nt < LM_T / 8; nt += 2) {
      if (nt < key_tiles) {                                // key_tiles is even
        uint32_t b[4];
        load_b_pair(b, ks_, LDD, nt * 8, kk, lane);
        mma_bf16(acc[nt], a, b[0], b[1]);
        mma_bf16(acc[nt + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < LM_T / 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = r0 + g + (i >= 2 ? 8 : 0), col = nt * 8 + 2 * t + (i & 1);
      const float w = (nt < key_tiles && col <= row) ? acc[nt][i] * pw[row - col] : 0.f;
      split_bf16(w, &p_hi[row * LDT + col], &p_lo[row * LDT + col]);
    }
  }
  __syncwarp();
  // the rows' outputs: intra-run part into acc, the part of the state in front of the run into acc_s
  float acc_s[LM_COLS / 8][4];
#pragma unroll
  for (int nt = 0; nt < LM_COLS / 8; ++nt) {
    acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    acc_s[nt][0] = acc_s[nt][1] = acc_s[nt][2] = acc_s[nt][3] = 0.f;
  }
  for (int ks = 0; ks <= warp; ++ks) {                  // key blocks of 16 up to the diagonal
    uint32_t ah[4], al[4];
    load_a(ah, p_hi, LDT, r0, ks * 16, lane);
    load_a(al, p_lo, LDT, r0, ks * 16, lane);
#pragma unroll
    for (int nt = 0; nt < LM_COLS / 8; nt += 2) {
      uint32_t b[4];
      load_b_pair(b, vt, LDT, nt * 8, ks * 16, lane);
      mma_bf16(acc[nt], ah, b[0], b[1]);
      mma_bf16(acc[nt], al, b[0], b[1]);
      mma_bf16(acc[nt + 1], ah, b[2], b[3]);
      mma_bf16(acc[nt + 1], al, b[2], b[3]);
    }
  }
  for (int kk = 0; kk < dim; kk += 16) {
    uint32_t a[4];
    load_a(a, qs, LDD, r0, kk, lane);
#pragma unroll
    for (int nt = 0; nt < LM_COLS / 8; nt += 2) {
      uint32_t bh[4], bl[4];
      load_b_pair(bh, st_hi, LDD, nt * 8, kk, lane);
      load_b_pair(bl, st_lo, LDD, nt * 8, kk, lane);
      mma_bf16(acc_s[nt], a, bh[0], bh[1]);
      mma_bf16(acc_s[nt], a, bl[0], bl[1]);
      mma_bf16(acc_s[nt + 1], a, bh[2], bh[3]);
      mma_bf16(acc_s[nt + 1], a, bl[2], bl[3]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < LM_COLS / 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = r0 + g + (i >= 2 ? 8 : 0), c = c0 + nt * 8 + 2 * t + (i & 1);
      if (row < n && c < vdim)
        out[(long long)(begin + t0 + row) * ld_o + (long long)head * vdim + c] = fmaf(pw[row + 1], acc_s[nt][i], acc[nt][i]);
    }
  }
}

size_t la_mma_out_smem(int dim) {
  return sizeof(bf16) * ((size_t)2 * LM_T * (dim + LM_PAD) + 2 * LM_COLS * (dim + LM_PAD) + LM_COLS * (LM_T + LM_PAD) +
                         2 * LM_T * (LM_T + LM_PAD)) + sizeof(float) * (LM_T + 1);
}

// key sizes in steps of 16, value sizes in steps of 8 and rows that 16-byte loads can read
bool la_mma_takes(int dim, int vdim, long long ld, const void* q, const void* k, const void* v) {
  return dim % 16 == 0 && vdim % 8 == 0 && dim <= LA_MAX_DIM && ld % 8 == 0 && la_mma_out_smem(dim) <= 200 * 1024 &&
         (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0;
}

int launch_chunked_mma(const void* q, const void* k, const void* v, long long ld, const float* decay, float* state,
                       const int* cu_tokens, const int* slots, float* out, long long ld_o, float* sums, int requests,
                       int tokens, int heads, int dim, int vdim, int activation, int write_state, cudaStream_t stream) {
  const unsigned tiles = (unsigned)((vdim + LM_COLS - 1) / LM_COLS);
  const dim3 grid(heads, (unsigned)(tokens / LM_T + requests), tiles);
  const size_t smem1 = sizeof(bf16) * ((size_t)2 * dim * (LM_T + LM_PAD) + LM_COLS * (LM_T + LM_PAD)) + sizeof(float) * (LM_T + 1);
  const size_t smem3 = la_mma_out_smem(dim);
  auto go = [&](auto sums_kernel, auto out_kernel) {
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (smem3 > 48 * 1024) cudaFuncSetAttribute(out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    hfee_launch(sums_kernel, grid, dim3(LM_WARPS * 32), smem1, stream, (const bf16*)k, (const bf16*)v, ld, decay, cu_tokens,
                sums, requests, heads, dim, vdim);
    const long long per = (long long)dim * vdim;
    const unsigned z = (unsigned)((per + 255) / 256 < 64 ? (per + 255) / 256 : 64);
    hfee_launch(la_chunk_scan_kernel<LM_T>, dim3(heads, requests, z), dim3(256), 0, stream, decay, cu_tokens, slots, sums,
                state, heads, dim, vdim, write_state);
    hfee_launch(out_kernel, grid, dim3(LM_WARPS * 32), smem3, stream, (const bf16*)q, (const bf16*)k, (const bf16*)v, ld,
                decay, cu_tokens, (const float*)sums, out, ld_o, requests, heads, dim, vdim);
  };
  if (activation == ACT_SILU) go(la_mma_sums_kernel<ACT_SILU>, la_mma_out_kernel<ACT_SILU>);
  else go(la_mma_sums_kernel<ACT_NONE>, la_mma_out_kernel<ACT_NONE>);
  return hfee_check_launch("linear_attention_chunked (tensor cores)");
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
    hfee_launch(la_chunk_scan_kernel<LC_T>, dim3(heads, requests, z), dim3(256), 0, stream, decay, cu_tokens, slots, sums, state,
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
                                           int write_state, int tensor_cores, cudaStream_t stream) {
  if (requests == 0 || tokens == 0) return HFEE_OK;
  if (int e = check_sizes("linear_attention_chunked", requests, heads, dim, vdim, ld, ld_o, activation)) return e;
  HFEE_REQUIRE(workspace != nullptr && workspace_floats >= hfee_linear_attention_chunked_workspace(requests, tokens, heads, dim, vdim),
               "linear_attention_chunked: the workspace is too small");
  if (dtype == HFEE_F32)
    return launch_chunked<float>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, workspace, requests, tokens, heads, dim, vdim, activation, write_state, stream);
  if (dtype == HFEE_BF16 && tensor_cores && la_mma_takes(dim, vdim, ld, q, k, v))
    return launch_chunked_mma(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, workspace, requests, tokens, heads, dim, vdim, activation, write_state, stream);
  if (dtype == HFEE_BF16)
    return launch_chunked<__nv_bfloat16>(q, k, v, ld, decay, state, cu_tokens, slots, out, ld_o, workspace, requests, tokens, heads, dim, vdim, activation, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "linear_attention_chunked: unknown dtype %d", dtype);
}
