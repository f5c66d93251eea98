// Causal depthwise convolution over time with a per-request history, added to its input:
//
//   out[t, c] = x[t, c] + sum_{j < taps} w[c, j] * x[t - taps + 1 + j, c]
//
// where t counts a request's tokens and inputs in front of the tokens of this step come from
// the request's state, the last taps - 1 inputs it has seen (zeros for a fresh request, which is
// what "zeros before the start of the sequence" asks for).  After the step the state holds the
// last taps - 1 inputs again.  Arithmetic is float32; x is the float32 residual stream, TOut the
// type the next matrix product reads.
//
// A thread owns one channel (two, when the width is even) of a run of SC_TOKENS tokens of one request and
// slides the window through registers.  The block that holds a request's last token writes the new state; when a
// portion is longer than one run, another block reads the old state at the same time, so the
// launcher then writes the state in a second launch.
#include "common.cuh"

namespace {

constexpr int SC_MAX_TAPS = 8;
constexpr int SC_TOKENS = 16;
constexpr int SC_THREADS = 128;
constexpr int SC_OUT = 1, SC_STATE = 2;

// CH = channels per thread: 2 (8-byte loads, 4-byte bfloat16 stores) for even widths, else 1.
template <int CH> struct Chan;
template <> struct Chan<1> {
  float v[1];
  __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
  __device__ __forceinline__ void zero() { v[0] = 0.f; }
};
template <> struct Chan<2> {
  float v[2];
  __device__ __forceinline__ void load(const float* p) { const float2 t = *reinterpret_cast<const float2*>(p); v[0] = t.x; v[1] = t.y; }
  __device__ __forceinline__ void zero() { v[0] = v[1] = 0.f; }
};
template <int CH> __device__ __forceinline__ void store_chan(float* p, const float (&v)[CH]) {
  if constexpr (CH == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); else p[0] = v[0];
}
template <int CH> __device__ __forceinline__ void store_chan(__nv_bfloat16* p, const float (&v)[CH]) {
  if constexpr (CH == 2) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]); else p[0] = __float2bfloat16_rn(v[0]);
}

template <typename TOut, int CH>
__global__ void __launch_bounds__(SC_THREADS)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ state,
                  const int* __restrict__ cu_tokens, const int* __restrict__ slots, TOut* __restrict__ out,
                  long long ld_out, int width, int taps, int mode) {
  const int req = blockIdx.y;
  const int c = (blockIdx.z * SC_THREADS + threadIdx.x) * CH;
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;     // host-written batch layout
  const int slot = slots[req];
  pdl_wait();
  pdl_launch_dependents();
  if (count <= 0 || c >= width) return;
  const int hist = taps - 1;
  // the state-only launch has one block per request: the run that holds the last token
  const int first = (mode == SC_STATE) ? ((count - 1) / SC_TOKENS) * SC_TOKENS : blockIdx.x * SC_TOKENS;
  if (first >= count) return;
  const int last = min(count, first + SC_TOKENS);
  float* st = state + (long long)slot * hist * width + c;                    // st[s * width]: input at index s - hist
  const float* xc = x + (long long)begin * width + c;

  float wv[CH][SC_MAX_TAPS];
  Chan<CH> win[SC_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS; ++j) {
#pragma unroll
    for (int k = 0; k < CH; ++k) wv[k][j] = j < taps ? w[(long long)(c + k) * taps + j] : 0.f;
    win[j].zero();
    if (j < hist) {
      const int s = first - hist + j;                                        // index within the portion
      win[j].load(s >= 0 ? xc + (long long)s * width : st + (long long)(hist + s) * width);
    }
  }
  if (mode & SC_OUT) {
    Chan<CH> xin[SC_TOKENS];                  // the run's inputs, requested together
#pragma unroll
    for (int i = 0; i < SC_TOKENS; ++i) {
      xin[i].zero();
      if (first + i < last) xin[i].load(xc + (long long)(first + i) * width);
    }
#pragma unroll
    for (int i = 0; i < SC_TOKENS; ++i) {
      const int t = first + i;
      if (t >= last) break;
      float o[CH];
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const float xv = xin[i].v[k];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < SC_MAX_TAPS; ++j) {
          const float in = (j == hist) ? xv : win[j].v[k];
          if (j < taps) acc = fmaf(wv[k][j], in, acc);
        }
        o[k] = xv + acc;
      }
      store_chan<CH>(out + (long long)(begin + t) * ld_out + c, o);
#pragma unroll
      for (int j = 0; j + 1 < SC_MAX_TAPS; ++j) win[j] = (j + 1 == hist) ? xin[i] : win[j + 1];
    }
  }
  if ((mode & SC_STATE) && last == count) {
    // new st[s] = input at index count - hist + s; a negative index lies in the old state, at a
    // higher place than the one being written, so ascending order reads before it overwrites
    for (int s = 0; s < hist; ++s) {
      const int idx = count - hist + s;
      Chan<CH> v;
      v.load(idx >= 0 ? xc + (long long)idx * width : st + (long long)(hist + idx) * width);
      store_chan<CH>(st + (long long)s * width, v.v);
    }
  }
}

template <typename TOut, int CH>
int launch_short_conv_ch(const float* x, const float* w, float* state, const int* cu_tokens, const int* slots, void* out,
                         long long ld_out, int requests, int max_new, int width, int taps, int write_state,
                         cudaStream_t stream) {
  const unsigned runs = (unsigned)((max_new + SC_TOKENS - 1) / SC_TOKENS);
  const unsigned cz = (unsigned)((width / CH + SC_THREADS - 1) / SC_THREADS);
  const bool together = write_state && runs == 1 && taps > 1;
  hfee_launch(short_conv_kernel<TOut, CH>, dim3(runs, requests, cz), dim3(SC_THREADS), 0, stream, x, w, state, cu_tokens,
              slots, (TOut*)out, ld_out, width, taps, together ? (SC_OUT | SC_STATE) : SC_OUT);
  if (write_state && !together && taps > 1)
    hfee_launch(short_conv_kernel<TOut, CH>, dim3(1, requests, cz), dim3(SC_THREADS), 0, stream, x, w, state, cu_tokens,
                slots, (TOut*)out, ld_out, width, taps, SC_STATE);
  return hfee_check_launch("short_conv");
}

template <typename TOut>
int launch_short_conv(const float* x, const float* w, float* state, const int* cu_tokens, const int* slots, void* out,
                      long long ld_out, int requests, int max_new, int width, int taps, int write_state,
                      cudaStream_t stream) {
  const bool pairs = width % 2 == 0 && ld_out % 2 == 0 && (uintptr_t)x % 8 == 0 && (uintptr_t)state % 8 == 0 &&
                     (uintptr_t)out % (2 * sizeof(TOut)) == 0;
  if (pairs)
    return launch_short_conv_ch<TOut, 2>(x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, write_state, stream);
  return launch_short_conv_ch<TOut, 1>(x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, write_state, stream);
}

}  // namespace

// Launches one kernel, or two when a portion is longer than one run of tokens and the state is written.
HFEE_API int hfee_short_conv_launches(int max_new, int taps, int write_state) {
  return (write_state && taps > 1 && max_new > SC_TOKENS) ? 2 : 1;
}

HFEE_API int hfee_short_conv(const float* x, const float* w, float* state, const int* cu_tokens, const int* slots,
                             void* out, long long ld_out, int out_dtype, int requests, int max_new, int width, int taps,
                             int write_state, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(requests > 0 && max_new > 0 && width > 0, "short_conv: bad sizes");
  HFEE_REQUIRE(taps >= 1 && taps <= SC_MAX_TAPS, "short_conv: taps %d is outside 1..%d", taps, SC_MAX_TAPS);
  HFEE_REQUIRE(ld_out >= width, "short_conv: ld_out=%lld is too small", ld_out);
  if (out_dtype == HFEE_F32)
    return launch_short_conv<float>(x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, write_state, stream);
  if (out_dtype == HFEE_BF16)
    return launch_short_conv<__nv_bfloat16>(x, w, state, cu_tokens, slots, out, ld_out, requests, max_new, width, taps, write_state, stream);
  return hfee_fail(HFEE_ERR_ARG, "short_conv: unknown dtype %d", out_dtype);
}
