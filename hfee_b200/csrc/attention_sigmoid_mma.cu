// Attention with unnormalised sigmoid weights over the paged cache on mma.sync tensor cores (bfloat16):
//
//   o[t, h] = gate * sum_j sigmoid((q[t, h] . k[j]) * scale * head_scale[h] + head_bias[h]) * v[j]
//
// over the keys j of the token's own request with lo(t) <= j <= pos(t), where lo(t) is the start of the
// block of `chunk` positions that holds pos(t) (chunk = 0: position 0) and not below pos(t) + 1 - window
// (window = 0: no window).  Nothing is normalised over the keys, so key blocks can be added in any order
// and no running maximum is kept.
//
// A CTA takes SA_ROWS / group consecutive tokens of one request and one key/value head: its rows are the
// (token, query head of the group) pairs, 16 per warp.  Keys run in blocks of 64 from lo(first token) to
// pos(last token): K rows and transposed V rows go to shared memory through the block table, scores are
// float32 sums of bfloat16 products, the weights are computed in float32 and enter the second product as the
// sum of two bfloat16 numbers (the weight rounded, and what the rounding left), so that they carry 16 bits.
// The same kernel serves prompt portions and decode steps (one token per request: the first warps have rows).
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int SA_ROWS = 64;       // rows of a CTA: (token, head of the group) pairs (128 rows on 8 warps measured the same at head 64, slower at 128)
constexpr int SA_WARPS = 4;
constexpr int SA_KEYS = 64;       // keys per block
constexpr int SA_PAD = 8;

template <int HD>
__global__ void __launch_bounds__(SA_WARPS * 32)
attention_sigmoid_mma_kernel(const bf16* __restrict__ q, long long ld_q, const bf16* __restrict__ k_pool,
                             const bf16* __restrict__ v_pool, PagedCache cache, const int* __restrict__ cu_tokens,
                             const int* __restrict__ slots, const int* __restrict__ context_before,
                             bf16* __restrict__ out, long long ld_o, int requests, int heads, float scale, int window,
                             int chunk, const float* __restrict__ head_scale, const float* __restrict__ head_bias,
                             const bf16* __restrict__ gate, long long ld_gate) {
  constexpr int LDD = HD + SA_PAD, LDK = SA_KEYS + SA_PAD, NT = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);        // [SA_ROWS][LDD]
  bf16* ks = qs + SA_ROWS * LDD;                       // [SA_KEYS][LDD]
  bf16* vt = ks + SA_KEYS * LDD;                       // [HD][LDK]      values transposed
  bf16* p_hi = vt + HD * LDK;                          // [SA_ROWS][LDK]
  bf16* p_lo = p_hi + SA_ROWS * LDK;
  const int group = heads / cache.kv_heads;
  const int tokens_per_cta = SA_ROWS / group;
  const int kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  // which request and which of its token tiles: tiles are numbered request by request
  int req = -1, tile = 0, base = 0;
  for (int r = 0; r < requests; ++r) {
    const int c = (cu_tokens[r + 1] - cu_tokens[r] + tokens_per_cta - 1) / tokens_per_cta;
    if ((int)blockIdx.x < base + c) { req = r; tile = blockIdx.x - base; break; }
    base += c;
  }
  if (req < 0) return;                                  // the grid is an upper bound of the number of tiles
  const int begin = cu_tokens[req], count = cu_tokens[req + 1] - begin;
  const int slot = slots[req], first_pos = context_before[req];
  const int tok0 = tile * tokens_per_cta, ntok = min(tokens_per_cta, count - tok0);
  const int rows = ntok * group;
  pdl_wait();
  pdl_launch_dependents();

  // 16-byte accesses: a thread takes 8 consecutive dimensions of a row
  for (int e = threadIdx.x; e < SA_ROWS * (HD / 8); e += SA_WARPS * 32) {
    const int r = e / (HD / 8), d = (e % (HD / 8)) * 8;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows)
      val = *reinterpret_cast<const uint4*>(q + (long long)(begin + tok0 + r / group) * ld_q + (long long)(kvh * group + r % group) * HD + d);
    *reinterpret_cast<uint4*>(qs + r * LDD + d) = val;
  }
  // positions and visibility of this thread's rows: r0 + g and r0 + g + 8
  const int r0 = warp * 16;
  int pos_row[2], lo_row[2];
  float hs[2], hb[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + g + 8 * i;
    const int p = first_pos + tok0 + min(r, rows - 1) / group;
    pos_row[i] = r < rows ? p : -1;                     // no key is visible to a row past the end
    int lo = chunk > 0 ? (p / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, p + 1 - window);
    lo_row[i] = lo;
    const int h = kvh * group + min(r, rows - 1) % group;
    hs[i] = scale * (head_scale != nullptr ? head_scale[h] : 1.f);
    hb[i] = head_bias != nullptr ? head_bias[h] : 0.f;
  }
  const int p_first = first_pos + tok0, p_last = p_first + ntok - 1;
  int key_lo = chunk > 0 ? (p_first / chunk) * chunk : 0;
  if (window > 0) key_lo = max(key_lo, p_first + 1 - window);

  // the keys this warp's sixteen rows can see at all: a key block outside [warp_lo, warp_hi] is skipped by the warp
  const int warp_hi = first_pos + tok0 + min(r0 + 15, rows - 1) / group;
  const int p_warp = first_pos + tok0 + min(r0, rows - 1) / group;
  int warp_lo = chunk > 0 ? (p_warp / chunk) * chunk : 0;
  if (window > 0) warp_lo = max(warp_lo, p_warp + 1 - window);

  float acc_o[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc_o[nt][0] = acc_o[nt][1] = acc_o[nt][2] = acc_o[nt][3] = 0.f;

  for (int kb = key_lo; kb <= p_last; kb += SA_KEYS) {
    __syncthreads();                                    // the block before is used up (and qs is written)
    for (int e = threadIdx.x; e < SA_KEYS * (HD / 8); e += SA_WARPS * 32) {
      const int j = e % SA_KEYS, d = (e / SA_KEYS) * 8;      // neighbouring threads: neighbouring keys (transposed stores meet no bank twice)
      uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = make_uint4(0u, 0u, 0u, 0u);
      if (kb + j <= p_last) {
        const long long at = paged_offset(cache, slot, kb + j, kvh) + d;
        kv = *reinterpret_cast<const uint4*>(k_pool + at);
        vv = *reinterpret_cast<const uint4*>(v_pool + at);
      }
      *reinterpret_cast<uint4*>(ks + j * LDD + d) = kv;
      const bf16* v8 = reinterpret_cast<const bf16*>(&vv);
#pragma unroll
      for (int i = 0; i < 8; ++i) vt[(d + i) * LDK + j] = v8[i];
    }
    __syncthreads();
    if (r0 < rows && kb <= warp_hi && kb + SA_KEYS > warp_lo) {
      float acc_s[SA_KEYS / 8][4];
#pragma unroll
      for (int nt = 0; nt < SA_KEYS / 8; ++nt) acc_s[nt][0] = acc_s[nt][1] = acc_s[nt][2] = acc_s[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD; kk += 16) {
        uint32_t a[4];
        load_a(a, qs, LDD, r0, kk, lane);
#pragma unroll
        for (int nt = 0; nt < SA_KEYS / 8; nt += 2) {
          uint32_t b[4];
          load_b_pair(b, ks, LDD, nt * 8, kk, lane);
          mma_bf16(acc_s[nt], a, b[0], b[1]);
          mma_bf16(acc_s[nt + 1], a, b[2], b[3]);
        }
      }
      // sigmoid by ex2.approx and a fast division (relative error about 2^-21, far below the 16 bits the weights
      // keep); a thread's two neighbouring keys are stored together
#pragma unroll
      for (int nt = 0; nt < SA_KEYS / 8; ++nt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float w[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int key = kb + nt * 8 + 2 * t4 + j;
            w[j] = (key >= lo_row[half] && key <= pos_row[half])
                       ? __fdividef(1.f, 1.f + __expf(-fmaf(acc_s[nt][2 * half + j], hs[half], hb[half]))) : 0.f;
          }
          const __nv_bfloat162 hi = __floats2bfloat162_rn(w[0], w[1]);
          const __nv_bfloat162 lo = __floats2bfloat162_rn(w[0] - __bfloat162float(hi.x), w[1] - __bfloat162float(hi.y));
          const int at = (r0 + g + 8 * half) * LDK + nt * 8 + 2 * t4;
          *reinterpret_cast<__nv_bfloat162*>(p_hi + at) = hi;
          *reinterpret_cast<__nv_bfloat162*>(p_lo + at) = lo;
        }
      }
      __syncwarp();
#pragma unroll
      for (int ks16 = 0; ks16 < SA_KEYS / 16; ++ks16) {
        uint32_t ah[4], al[4];
        load_a(ah, p_hi, LDK, r0, ks16 * 16, lane);
        load_a(al, p_lo, LDK, r0, ks16 * 16, lane);
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t b[4];
          load_b_pair(b, vt, LDK, nt * 8, ks16 * 16, lane);
          mma_bf16(acc_o[nt], ah, b[0], b[1]);
          mma_bf16(acc_o[nt], al, b[0], b[1]);
          mma_bf16(acc_o[nt + 1], ah, b[2], b[3]);
          mma_bf16(acc_o[nt + 1], al, b[2], b[3]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r0 + g + 8 * half;
    if (r >= rows) continue;
    const long long token = begin + tok0 + r / group;
    const int h = kvh * group + r % group;
    bf16* orow = out + token * ld_o + (long long)h * HD;
    const bf16* grow = gate != nullptr ? gate + token * ld_gate + (long long)h * HD : nullptr;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int d = nt * 8 + 2 * t4;
      float o0 = acc_o[nt][2 * half], o1 = acc_o[nt][2 * half + 1];
      if (grow != nullptr) {
        const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(grow + d);
        o0 *= __fdividef(1.f, 1.f + __expf(-__bfloat162float(g2.x)));
        o1 *= __fdividef(1.f, 1.f + __expf(-__bfloat162float(g2.y)));
      }
      *reinterpret_cast<__nv_bfloat162*>(orow + d) = __floats2bfloat162_rn(o0, o1);
    }
  }
}

template <int HD>
int launch_sigmoid_mma(const void* q, long long ld_q, const void* k_pool, const void* v_pool, const PagedCache& c,
                       const int* cu_tokens, const int* slots, const int* context_before, void* out, long long ld_o,
                       int n_tokens, int requests, int heads, float scale, int window, int chunk, const float* head_scale,
                       const float* head_bias, const void* gate, long long ld_gate, cudaStream_t stream) {
  const int group = heads / c.kv_heads, per = SA_ROWS / group;
  const size_t smem = sizeof(bf16) * ((size_t)(SA_ROWS + SA_KEYS) * (HD + SA_PAD) + (HD + 2 * SA_ROWS) * (SA_KEYS + SA_PAD));
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attention_sigmoid_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const dim3 grid((unsigned)(n_tokens / per + requests), (unsigned)c.kv_heads);
  hfee_launch(attention_sigmoid_mma_kernel<HD>, grid, dim3(SA_WARPS * 32), smem, stream, (const bf16*)q, ld_q,
              (const bf16*)k_pool, (const bf16*)v_pool, c, cu_tokens, slots, context_before, (bf16*)out, ld_o, requests,
              heads, scale, window, chunk, head_scale, head_bias, (const bf16*)gate, ld_gate);
  return hfee_check_launch("attention_sigmoid_mma");
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes: a head size it is built for, a group that divides its rows,
// rows of q, out and gate that 4-byte accesses can read.
HFEE_API int hfee_attention_sigmoid_mma_supports(int heads, int kv_heads, int head_dim) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
  const int group = heads / kv_heads;
  if (group > SA_ROWS || SA_ROWS % group) return 0;
  return head_dim == 16 || head_dim == 32 || head_dim == 48 || head_dim == 64 || head_dim == 96 || head_dim == 128;
}

HFEE_API int hfee_attention_sigmoid_mma(const void* q, long long ld_q, const void* k_pool, const void* v_pool,
                                        const int* block_table, int max_pages, int page_size, const int* cu_tokens,
                                        const int* slots, const int* context_before, void* out, long long ld_o,
                                        int n_tokens, int requests, int heads, int kv_heads, int head_dim, float scale,
                                        int window, int chunk, const float* head_scale, const float* head_bias,
                                        const void* gate, long long ld_gate, cudaStream_t stream) {
  if (n_tokens == 0 || requests == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_attention_sigmoid_mma_supports(heads, kv_heads, head_dim),
               "attention_sigmoid_mma: heads %d, kv_heads %d, head_dim %d are not sizes of this kernel", heads, kv_heads, head_dim);
  HFEE_REQUIRE(ld_q % 8 == 0 && (uintptr_t)q % 16 == 0, "attention_sigmoid_mma: query rows must start on 16-byte boundaries");
  HFEE_REQUIRE(ld_o % 2 == 0 && (gate == nullptr || ld_gate % 2 == 0) && (uintptr_t)out % 4 == 0 && (uintptr_t)gate % 4 == 0,
               "attention_sigmoid_mma: output and gate rows must start on 4-byte boundaries");
  HFEE_REQUIRE(window >= 0 && chunk >= 0, "attention_sigmoid_mma: bad mask option");
  PagedCache c;
  HFEE_REQUIRE(make_paged_cache(&c, block_table, max_pages, page_size, kv_heads, head_dim),
               "page_size %d must be a power of two", page_size);
#define HFEE_SA_GO(HD)                                                                                              \
  case HD:                                                                                                          \
    return launch_sigmoid_mma<HD>(q, ld_q, k_pool, v_pool, c, cu_tokens, slots, context_before, out, ld_o, n_tokens, \
                                  requests, heads, scale, window, chunk, head_scale, head_bias, gate, ld_gate, stream)
  switch (head_dim) {
    HFEE_SA_GO(16); HFEE_SA_GO(32); HFEE_SA_GO(48); HFEE_SA_GO(64); HFEE_SA_GO(96); HFEE_SA_GO(128);
  }
#undef HFEE_SA_GO
  return hfee_fail(HFEE_ERR_ARG, "attention_sigmoid_mma: head_dim %d", head_dim);
}
