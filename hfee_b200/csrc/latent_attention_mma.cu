// Softmax attention of many query heads over ONE cached vector per token whose leading dimensions are also the
// values (a latent attention's cache: [normed latent | rotated shared key part]), on bfloat16 tensor-core MMAs
// (mma.sync.m16n8k16) with float32 scores and a float32 online softmax, for prompt portions, single decoded
// tokens and mixtures of both in one launch.
//
// All heads of a token read the same keys, so the rows of a tile are (token, head) pairs: a CTA serves
// LA_ROWS rows of one request (several tokens when there are few heads, a slice of the heads when there are many).
// Keys are visited in blocks of LA_BN positions aligned to absolute multiples of LA_BN, fetched row by row through the
// block table with cp.async into one of two buffers while the block before is being used; rows outside the tile's key range
// are zero-filled so that stale page content (or a page the window has given back) never reaches an MMA.
// The key size (hundreds of dimensions) is too large to keep queries or outputs of 16 rows in one warp's
// registers, so the four warps split a block twice: for S = Q K^T each warp takes 16 of the block's keys (queries
// and keys both come from shared memory), the row maxima and sums meet in shared memory, the weights go to shared
// memory as bfloat16, and for O += P V each warp takes every fourth group of 16 value columns for all rows.
#include "mma_tiles.cuh"

namespace {

constexpr int LA_ROWS = 32;
constexpr int LA_BN = 64;
constexpr int LA_WARPS = 4;
constexpr int LA_THREADS = LA_WARPS * 32;
constexpr int LA_PAD = 8;
constexpr int LA_PS_LD = LA_BN + LA_PAD;

struct LatentParams {
  const bf16* q; long long ld_q;
  bf16* out; long long ld_o;
  const bf16* pool;                // [pages][1][page_size][dk]
  const int* block_table; int max_pages, page_shift, page_mask;
  const int* cu_tokens; const int* slots; const int* context_before;
  int heads, dk, dv;
  int rows_per_token, tokens_per_tile;
  float scale_log2;
  int window;
};

__device__ __forceinline__ void la_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void la_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void la_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void la_ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ float la_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NG: groups of 16 value columns per warp (dv <= 64 * NG).  WG: sets of four warps; each set owns LA_ROWS rows of the
// tile and works as described above, and all sets share the key blocks in shared memory (half the cache traffic per row
// and twice the warps per block with two sets).
template <int NG, int WG>
__global__ void __launch_bounds__(LA_THREADS * WG)
latent_attention_kernel(LatentParams p) {
  constexpr int ROWS = LA_ROWS * WG, THREADS = LA_THREADS * WG;
  extern __shared__ __align__(16) unsigned char la_smem[];
  const int dk = p.dk, dv = p.dv, ldk = dk + LA_PAD;
  bf16* Qs = reinterpret_cast<bf16*>(la_smem);                // [LA_ROWS][ldk]
  bf16* Ks = Qs + ROWS * ldk;                                 // [2][LA_BN][ldk]
  bf16* Ps = Ks + 2 * LA_BN * ldk;                            // [ROWS][LA_PS_LD]
  float* m_s = reinterpret_cast<float*>(Ps + ROWS * LA_PS_LD);
  float* l_s = m_s + ROWS;
  float* wmax = l_s + ROWS;                                   // [LA_WARPS][ROWS]
  float* wsum = wmax + LA_WARPS * ROWS;                       // [LA_WARPS][ROWS]
  int* rowpos = reinterpret_cast<int*>(wsum + LA_WARPS * ROWS);      // position of the row's token, -1: no row

  const int req = blockIdx.z, head0 = blockIdx.y * p.rows_per_token;
  const int begin = p.cu_tokens[req], count = p.cu_tokens[req + 1] - begin;     // host-written batch layout
  const int t0 = blockIdx.x * p.tokens_per_tile;
  pdl_wait();
  pdl_launch_dependents();
  if (t0 >= count) return;
  const int tokens = min(p.tokens_per_tile, count - t0);
  const int slot = p.slots[req], before = p.context_before[req];
  const int tid = threadIdx.x, warp = (tid >> 5) % LA_WARPS, lane = tid & 31;
  const int rb = (tid >> 5) / LA_WARPS * LA_ROWS;              // first row of this set of warps
  const int p_first = before + t0, p_last = before + t0 + tokens - 1;
  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
  const int* table = p.block_table + (long long)slot * p.max_pages;
  const long long page_stride = (long long)(p.page_mask + 1) * dk;

  if (tid < ROWS) {
    const int t = tid / p.rows_per_token, h = head0 + tid % p.rows_per_token;
    rowpos[tid] = (t < tokens && h < p.heads) ? before + t0 + t : -1;
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  // queries of the tile
  const int pieces = dk >> 3;
  for (int e = tid; e < ROWS * pieces; e += THREADS) {
    const int r = e / pieces, c = (e - r * pieces) * 8;
    const int t = r / p.rows_per_token, h = head0 + r % p.rows_per_token;
    const bool valid = t < tokens && h < p.heads;
    const bf16* src = p.q + (long long)(begin + t0 + (valid ? t : 0)) * p.ld_q + (long long)(valid ? h : 0) * dk + c;
    la_cp_async16(Qs + r * ldk + c, src, valid);
  }
  auto load_block = [&](int block_start, int buf) {
    bf16* dst = Ks + (long long)buf * LA_BN * ldk;
    for (int e = tid; e < LA_BN * pieces; e += THREADS) {
      const int r = e / pieces, c = (e - r * pieces) * 8;
      const int kp = block_start + r;
      const bool valid = kp >= lo && kp <= p_last;
      const bf16* src = p.pool;
      if (valid) src += (long long)table[kp >> p.page_shift] * page_stride + (long long)(kp & p.page_mask) * dk + c;
      la_cp_async16(dst + r * ldk + c, src, valid);
    }
  };
  const int first_block = (lo / LA_BN) * LA_BN;
  load_block(first_block, 0);
  la_commit();

  float o[NG][2][2][4];          // [group][column tile of 8][row tile of 16][fragment]
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[g][a][b][c] = 0.f;
  const int groups = dv >> 4;
  const int quad_row = lane >> 2, quad_col = 2 * (lane & 3);

  int buf = 0;
  for (int block_start = first_block; block_start <= p_last; block_start += LA_BN, buf ^= 1) {
    la_wait_all();
    __syncthreads();
    if (block_start + LA_BN <= p_last) load_block(block_start + LA_BN, buf ^ 1);
    la_commit();
    const bf16* Kb = Ks + (long long)buf * LA_BN * ldk;

    // S = Q K^T for this warp's 16 keys: [2 row tiles][2 key tiles]
    float s[2][2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[a][b][c] = 0.f;
    for (int k0 = 0; k0 < dk; k0 += 16) {
      uint32_t a0[4], a1[4], b[4];
      load_a(a0, Qs, ldk, rb, k0, lane);
      load_a(a1, Qs, ldk, rb + 16, k0, lane);
      load_b_pair(b, Kb, ldk, 16 * warp, k0, lane);
      mma_bf16(s[0][0], a0, b[0], b[1]);
      mma_bf16(s[0][1], a0, b[2], b[3]);
      mma_bf16(s[1][0], a1, b[0], b[1]);
      mma_bf16(s[1][1], a1, b[2], b[3]);
    }
    // scale, mask, row maxima over the warp's keys
    float rmax[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int pos = rowpos[rb + mt * 16 + quad_row + 8 * half];
        const int low = p.window > 0 ? pos - p.window + 1 : 0;
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kp = block_start + 16 * warp + 8 * nt + quad_col + e;
            float v = s[mt][nt][2 * half + e] * p.scale_log2;
            if (kp > pos || kp < low) v = -INFINITY;
            s[mt][nt][2 * half + e] = v;
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        rmax[mt][half] = mx;
        if ((lane & 3) == 0) wmax[warp * ROWS + rb + mt * 16 + quad_row + 8 * half] = mx;
      }
    __syncthreads();
    // weights against the new row maximum; the factor the old sums and outputs shrink by
    float alpha[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = rb + mt * 16 + quad_row + 8 * half;
        const float m_old = m_s[row];
        float m_new = m_old;
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) m_new = fmaxf(m_new, wmax[w * ROWS + row]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        alpha[mt][half] = la_exp2(m_old - m_use);           // 2^-inf = 0 while the row has seen no key
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float p0 = la_exp2(s[mt][nt][2 * half] - m_use), p1 = la_exp2(s[mt][nt][2 * half + 1] - m_use);
          const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          // the sum runs over the rounded weights, which are what multiplies the values
          sum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
          *reinterpret_cast<__nv_bfloat162*>(Ps + row * LA_PS_LD + 16 * warp + 8 * nt + quad_col) = pb;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) wsum[warp * ROWS + row] = sum;
      }
    __syncthreads();
    if (tid < ROWS) {
      const float m_old = m_s[tid];
      float m_new = m_old, sum = 0.f;
#pragma unroll
      for (int w = 0; w < LA_WARPS; ++w) {
        m_new = fmaxf(m_new, wmax[w * ROWS + tid]);
        sum += wsum[w * ROWS + tid];
      }
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      l_s[tid] = l_s[tid] * la_exp2(m_old - m_use) + sum;
      m_s[tid] = m_new;
    }
    // O = alpha O + P V for this warp's value columns
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const int grp = warp + LA_WARPS * g;
      if (grp >= groups) break;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          o[g][nt][mt][0] *= alpha[mt][0];
          o[g][nt][mt][1] *= alpha[mt][0];
          o[g][nt][mt][2] *= alpha[mt][1];
          o[g][nt][mt][3] *= alpha[mt][1];
        }
#pragma unroll
      for (int k0 = 0; k0 < LA_BN; k0 += 16) {
        uint32_t a0[4], a1[4], b[4];
        load_a(a0, Ps, LA_PS_LD, rb, k0, lane);
        load_a(a1, Ps, LA_PS_LD, rb + 16, k0, lane);
        la_ldmatrix_x4_trans(b, Kb + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldk + 16 * grp + (lane >> 4) * 8);
        mma_bf16(o[g][0][0], a0, b[0], b[1]);
        mma_bf16(o[g][1][0], a0, b[2], b[3]);
        mma_bf16(o[g][0][1], a1, b[0], b[1]);
        mma_bf16(o[g][1][1], a1, b[2], b[3]);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = rb + mt * 16 + quad_row + 8 * half;
      if (rowpos[row] < 0) continue;
      const int t = row / p.rows_per_token, h = head0 + row % p.rows_per_token;
      const float l = l_s[row];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (long long)(begin + t0 + t) * p.ld_o + (long long)h * dv;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const int grp = warp + LA_WARPS * g;
        if (grp >= groups) break;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          *reinterpret_cast<__nv_bfloat162*>(dst + 16 * grp + 8 * nt + quad_col) =
              __floats2bfloat162_rn(o[g][nt][mt][2 * half] * inv, o[g][nt][mt][2 * half + 1] * inv);
      }
    }
}

size_t latent_smem(int dk, int rows) {
  return (size_t)(rows + 2 * LA_BN) * (dk + LA_PAD) * sizeof(bf16) + (size_t)rows * LA_PS_LD * sizeof(bf16) +
         (size_t)(2 + 2 * LA_WARPS) * rows * sizeof(float) + rows * sizeof(int);
}

template <int NG, int WG>
int launch_latent(const LatentParams& p, dim3 grid, cudaStream_t stream) {
  const size_t smem = latent_smem(p.dk, LA_ROWS * WG);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<NG, WG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "latent_attention_mma: %s", cudaGetErrorString(e));
  }
  hfee_launch(latent_attention_kernel<NG, WG>, grid, dim3(LA_THREADS * WG), smem, stream, p);
  return hfee_check_launch("latent_attention_mma");
}

}  // namespace

// 1 if the kernel takes these sizes: key size a multiple of 16 that fits shared memory, value size a multiple of 16
// of at most 512 and at most the key size.
HFEE_API int hfee_latent_attention_mma_supports(int heads, int dk, int dv) {
  return heads > 0 && dk > 0 && dk % 16 == 0 && dv > 0 && dv % 16 == 0 && dv <= dk && dv <= 512 && latent_smem(dk, LA_ROWS) <= 227 * 1024;
}

HFEE_API int hfee_latent_attention_mma(const void* q, long long ld_q, const void* pool, const int* block_table, int max_pages,
                                       int page_size, const int* cu_tokens, const int* slots, const int* context_before,
                                       void* out, long long ld_o, int requests, int max_new, int heads, int dk, int dv,
                                       float scale, int window, cudaStream_t stream) {
  if (requests == 0 || max_new == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_latent_attention_mma_supports(heads, dk, dv), "latent_attention_mma: sizes %d heads, %d key, %d value dimensions are not taken", heads, dk, dv);
  HFEE_REQUIRE(page_size > 0 && (page_size & (page_size - 1)) == 0, "page_size %d must be a power of two", page_size);
  HFEE_REQUIRE(ld_q % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)pool % 16 == 0, "latent_attention_mma: queries and cache must be 16-byte aligned");
  HFEE_REQUIRE(ld_o % 2 == 0 && (uintptr_t)out % 4 == 0, "latent_attention_mma: the output's rows must start on 4 bytes");
  HFEE_REQUIRE(requests <= 65535 && window >= 0, "latent_attention_mma: bad batch or window");
  LatentParams p{};
  p.q = (const bf16*)q; p.ld_q = ld_q; p.out = (bf16*)out; p.ld_o = ld_o; p.pool = (const bf16*)pool;
  p.block_table = block_table; p.max_pages = max_pages; p.page_mask = page_size - 1;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.cu_tokens = cu_tokens; p.slots = slots; p.context_before = context_before;
  p.heads = heads; p.dk = dk; p.dv = dv;
  // two sets of warps where their rows can be filled (several tokens of a portion, or many heads) and fit shared memory
  const int sets = ((long long)max_new * heads >= 2 * LA_ROWS && latent_smem(dk, 2 * LA_ROWS) <= 227 * 1024) ? 2 : 1;
  const int rows = LA_ROWS * sets;
  p.rows_per_token = heads < rows ? heads : rows;
  p.tokens_per_tile = rows / p.rows_per_token;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  const dim3 grid((unsigned)((max_new + p.tokens_per_tile - 1) / p.tokens_per_tile),
                  (unsigned)((heads + p.rows_per_token - 1) / p.rows_per_token), (unsigned)requests);
  HFEE_REQUIRE(grid.y <= 65535, "latent_attention_mma: too many heads");
  const int per_warp = (dv / 16 + LA_WARPS - 1) / LA_WARPS;
  if (sets == 2) {
    if (per_warp <= 1) return launch_latent<1, 2>(p, grid, stream);
    if (per_warp <= 2) return launch_latent<2, 2>(p, grid, stream);
    if (per_warp <= 4) return launch_latent<4, 2>(p, grid, stream);
    return launch_latent<8, 2>(p, grid, stream);
  }
  if (per_warp <= 1) return launch_latent<1, 1>(p, grid, stream);
  if (per_warp <= 2) return launch_latent<2, 1>(p, grid, stream);
  if (per_warp <= 4) return launch_latent<4, 1>(p, grid, stream);
  return launch_latent<8, 1>(p, grid, stream);
}
