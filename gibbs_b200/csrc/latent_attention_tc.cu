// Attention over a latent cache on tensor cores, in the absorbed form, for steps that carry portions of prompts.
//
// Every head's keys AND values are the same cached rows [c_j | k_rot,j] (kv_rank + rot_dim entries, bfloat16; the
// rotated part may be absent): with q'_h = [W_uk,h^T q_h | rot(q_rot,h)] the score is q'_h . [c_j | k_rot,j] and the
// head's output is sum_j p_j c_j: the first product reads whole rows, the second their first kv_rank entries.  So the rows of a tile are (token, head) pairs of one
// request, all of which read the same key rows, and one tile of cached rows in shared memory is the second operand of
// both products: S = Q' C^T (rows of C as they lie) and O += P C (the same rows, transposed on the way to the
// registers).
//
//  CTA: 64 rows = TPT consecutive tokens of one request x all heads (TPT = 64 / heads, rounded down), 4 warps of 16
//  rows; where the latent is wider than 256, a second group of 4 warps takes the other half of O's columns and
//  computes the same S (O of 16 x 256 is 128 registers a thread).  Key tiles of 64 rows arrive by cp.async through
//  the block table into two buffers.  mma.sync.m16n8k16, bfloat16 operands, 32-bit accumulators; the softmax (base
//  2, running maximum and sum per row) is 32-bit, and its weights enter the second product as TWO bfloat16 terms
//  (p = hi + lo), so 16 bits of every weight count.  A learned sink per head joins the denominator at the end; an
//  optional gate multiplies the result.  With `splits` 2 (a step of few tiles: one long prompt) the key tiles of
//  every row tile are cut in two halves for two CTAs, which leave (maximum, sum, weighted sum) per row for the merge
//  kernel of latent_attention.cu, and the row tiles with the most keys are launched first.  Causal, no window: what has one runs on the generic kernel, as do 32-bit
//  pages and steps of single tokens.  Rows in shared memory lie `stride` entries apart: the row's length rounded up
//  to 16, plus 8 (an odd number of 16-byte pieces, so that ldmatrix meets no bank twice).
#include "hybrid.cuh"

namespace {

enum { LTC_BAD_PAGE_READ = 2 };
#ifndef LTC_SPLIT_KEYS
#define LTC_SPLIT_KEYS 1
#endif
constexpr int LTC_ROWS = 64, LTC_KEYS = 64;

__device__ __forceinline__ void ltc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void ltc_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}
__device__ __forceinline__ void ltc_ldmatrix(unsigned (&r)[4], const bf16* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ltc_ldmatrix_t(unsigned (&r)[4], const bf16* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ltc_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ltc_pack(float x, float y) {
  __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<unsigned*>(&v);
}
// (hi, lo) of two weights: hi the nearest bfloat16, lo the nearest bfloat16 of what is left
__device__ __forceinline__ void ltc_split(float x, float y, unsigned& hi, unsigned& lo) {
  const bf16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
  __nv_bfloat162 h;
  h.x = hx;
  h.y = hy;
  hi = *reinterpret_cast<unsigned*>(&h);
  lo = ltc_pack(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

struct LtcParams {
  const float* qp;          // [tokens][heads][dk]
  const bf16* pages;        // [n_pages][page_size][dk]
  const int* block_table;
  int bt_stride, page_size, n_pages;
  const int* tok_req;
  const int* tok_pos;
  const int* q_start;      // first row per request; a request's rows end where the next one's begin
  int n, R;
  const float* gate;
  long long ld_gate;
  float* out;
  long long ldo;
  int H, r, tpt;
  int dk, stride;           // entries of a cached row (r + rotated part); entries between rows in shared memory
  int splits;               // 1, or 2: blockIdx.z takes one half of a row tile's key tiles and writes partial results
  float* ws;                // [tokens * heads][splits][r + 2] partial results (splits > 1)
  float scale_log2;
  const float* sink;
  int* status;
};

template <int RP>
__global__ void __launch_bounds__(RP > 256 ? 256 : 128, 1) latent_attention_tc_kernel(const LtcParams p) {
  constexpr int NSPLIT = RP > 256 ? 2 : 1, OC = RP / NSPLIT, THREADS = 128 * NSPLIT;
  const int STRIDE = p.stride, dk = p.dk;
  extern __shared__ __align__(16) unsigned char ltc_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(ltc_smem);           // [64][STRIDE]
  bf16* Cs = Qs + LTC_ROWS * STRIDE;                       // [2][64][STRIDE]
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = warp & 3, wn = warp >> 2;
  const int g = lane >> 2, t4 = lane & 3;
  const int req = blockIdx.y;
  const int first = p.q_start[req], len = (req + 1 < p.R ? p.q_start[req + 1] : p.n) - first;
  // (the row tiles with the most keys go first: where the grid is more than a wave, the short ones fill the end)
  const int tok0 = (int)(gridDim.x - 1 - blockIdx.x) * p.tpt;
  if (tok0 >= len) return;
  const int ntok = min(p.tpt, len - tok0), H = p.H, r = p.r;
  const int rows_live = ntok * H;
  const int t_first = first + tok0;
  const int pos0 = p.tok_pos[t_first];
  const int kmax = pos0 + ntok - 1;
  const int* table = p.block_table + (size_t)p.tok_req[t_first] * p.bt_stride;
  // zeros where nothing is copied: rows beyond the live ones, columns dk .. stride
  for (int i = threadIdx.x; i < 3 * LTC_ROWS * STRIDE / 8; i += THREADS)
    reinterpret_cast<uint4*>(ltc_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();

  const int pieces = dk >> 3;                              // 16-byte pieces of a cached row
  auto stage = [&](int kt, int b) {
    bf16* dst = Cs + (size_t)b * LTC_KEYS * STRIDE;
    for (int j = warp; j < LTC_KEYS; j += THREADS / 32) {
      const int key = min(kt * LTC_KEYS + j, kmax);         // (rows behind the last visible key are masked)
      int page = table[key / p.page_size];
      if (page < 0 || page >= p.n_pages) {
        if (lane == 0) atomicExch(p.status, LTC_BAD_PAGE_READ);
        continue;                                          // (the row keeps what it had: zeros or an older row)
      }
      const bf16* src = p.pages + ((size_t)page * p.page_size + key % p.page_size) * dk;
      for (int c = lane; c < pieces; c += 32) gb_cp_async_16(dst + j * STRIDE + 8 * c, src + 8 * c);
    }
    ltc_commit();
  };
  const int tiles = kmax / LTC_KEYS + 1;
  const int half_tiles = (tiles + 1) >> 1;
  const int kt_begin = p.splits > 1 ? (int)blockIdx.z * half_tiles : 0;
  const int kt_end = p.splits > 1 ? min(tiles, kt_begin + half_tiles) : tiles;
  pdl_wait();
  if (kt_begin < kt_end) stage(kt_begin, 0);
  {
    // this tile's queries: rows_live consecutive rows of dk floats, rounded to bfloat16
    const float* src = p.qp + (size_t)t_first * H * dk;
    const int quads = dk >> 2;
    for (int row = warp; row < rows_live; row += THREADS / 32)
      for (int c = lane; c < quads; c += 32) {
        const float4 v = *reinterpret_cast<const float4*>(src + (size_t)row * dk + 4 * c);
        uint2 w;
        w.x = ltc_pack(v.x, v.y);
        w.y = ltc_pack(v.z, v.w);
        *reinterpret_cast<uint2*>(Qs + row * STRIDE + 4 * c) = w;
      }
  }
  // this thread's two rows: wm * 16 + g and + 8
  const int row_a = wm * 16 + g, row_b = row_a + 8;
  const int tl_a = row_a / H, tl_b = row_b / H;
  const int h_a = row_a - tl_a * H, h_b = row_b - tl_b * H;
  const int pos_a = pos0 + tl_a, pos_b = pos0 + tl_b;
  const bool warp_live = wm * 16 < rows_live;

  float o[OC / 8][4];
#pragma unroll
  for (int j = 0; j < OC / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int ksteps = (dk + 15) >> 4;                       // k-steps of the first product that hold anything
  const int npairs = min(OC / 16, max(0, (r - wn * OC + 15) >> 4));   // pairs of 8 output columns likewise

  if (kt_begin >= kt_end) __syncthreads();                 // (the queries and zeros are written; no key tile follows)
  for (int kt = kt_begin; kt < kt_end; ++kt) {
    const int b = (kt - kt_begin) & 1;
    if (kt + 1 < kt_end) {
      stage(kt + 1, b ^ 1);
      ltc_wait<1>();
    } else {
      ltc_wait<0>();
    }
    __syncthreads();
    if (warp_live) {
      const bf16* C = Cs + (size_t)b * LTC_KEYS * STRIDE;
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const bf16* qa = Qs + (wm * 16 + (lane & 15)) * STRIDE + (lane >> 4) * 8;
      const bf16* cb = C + ((lane & 7) + (lane >> 4) * 8) * STRIDE + ((lane >> 3) & 1) * 8;
#pragma unroll 2
      for (int ks = 0; ks < ksteps; ++ks) {
        unsigned a[4];
        ltc_ldmatrix(a, qa + ks * 16);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          unsigned bb[4];
          ltc_ldmatrix(bb, cb + np * 16 * STRIDE + ks * 16);
          ltc_mma(s[2 * np], a, bb[0], bb[1]);
          ltc_mma(s[2 * np + 1], a, bb[2], bb[3]);
        }
      }
      // scores in base 2, the causal mask, the running maximum
      const int key0 = kt * LTC_KEYS + 2 * t4;
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = key0 + 8 * j;
        s[j][0] = k <= pos_a ? s[j][0] * p.scale_log2 : -INFINITY;
        s[j][1] = k + 1 <= pos_a ? s[j][1] * p.scale_log2 : -INFINITY;
        s[j][2] = k <= pos_b ? s[j][2] * p.scale_log2 : -INFINITY;
        s[j][3] = k + 1 <= pos_b ? s[j][3] * p.scale_log2 : -INFINITY;
        mx_a = fmaxf(mx_a, fmaxf(s[j][0], s[j][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[j][2], s[j][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      // (a row of a later token may see no key of this tile's first rows only if the tile lies behind it, and
      // such tiles are not visited by a CTA whose last token is that far; key 0 is visible to every row, so after
      // the first tile the maxima are finite.  A dead row of a partly filled tile has a clamped position.)
      const float ref_a = mn_a == -INFINITY ? 0.f : mn_a, ref_b = mn_b == -INFINITY ? 0.f : mn_b;
      const float corr_a = exp2f(m_a - ref_a), corr_b = exp2f(m_b - ref_b);
      m_a = mn_a;
      m_b = mn_b;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[j][0] = exp2f(s[j][0] - ref_a);
        s[j][1] = exp2f(s[j][1] - ref_a);
        s[j][2] = exp2f(s[j][2] - ref_b);
        s[j][3] = exp2f(s[j][3] - ref_b);
        sum_a += s[j][0] + s[j][1];
        sum_b += s[j][2] + s[j][3];
      }
      l_a = l_a * corr_a + sum_a;                          // (this lane's share; the quad is added at the end)
      l_b = l_b * corr_b + sum_b;
#pragma unroll
      for (int j = 0; j < OC / 8; ++j) {
        o[j][0] *= corr_a;
        o[j][1] *= corr_a;
        o[j][2] *= corr_b;
        o[j][3] *= corr_b;
      }
      // O += P C, the weights as hi + lo
      const bf16* ct = C + ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + wn * OC + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        unsigned hi[4], lo[4];
        ltc_split(s[2 * kk][0], s[2 * kk][1], hi[0], lo[0]);
        ltc_split(s[2 * kk][2], s[2 * kk][3], hi[1], lo[1]);
        ltc_split(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lo[2]);
        ltc_split(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lo[3]);
#pragma unroll
        for (int np = 0; np < OC / 16; ++np) {
          if (np < npairs) {
            unsigned bb[4];
            ltc_ldmatrix_t(bb, ct + kk * 16 * STRIDE + np * 16);
            ltc_mma(o[2 * np], hi, bb[0], bb[1]);
            ltc_mma(o[2 * np], lo, bb[0], bb[1]);
            ltc_mma(o[2 * np + 1], hi, bb[2], bb[3]);
            ltc_mma(o[2 * np + 1], lo, bb[2], bb[3]);
          }
        }
      }
    }
    __syncthreads();                                       // before the tile after next lands in this buffer
  }
  if (!warp_live) return;
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  constexpr float LOG2E = 1.4426950408889634f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? row_b : row_a;
    if (row >= rows_live) continue;
    const int tl = half ? tl_b : tl_a, h = half ? h_b : h_a;
    const float m = half ? m_b : m_a, l = half ? l_b : l_a;
    const size_t t = (size_t)t_first + tl;
    if (p.splits > 1) {
      // this half's partial result: maximum (natural units), sum of weights, weighted sum, for the merge kernel
      float* w = p.ws + ((t * H + h) * p.splits + blockIdx.z) * (size_t)(r + 2);
      if (wn == 0 && t4 == 0) {
        w[0] = m * 0.6931471805599453f;                    // (-inf stays -inf: a half without keys)
        w[1] = l;
      }
#pragma unroll
      for (int j = 0; j < OC / 8; ++j) {
        const int col = wn * OC + 8 * j + 2 * t4;
        if (col < r) {
          w[2 + col] = o[j][2 * half];
          w[2 + col + 1] = o[j][2 * half + 1];
        }
      }
      continue;
    }
    float f = 1.f / l;
    if (p.sink) {
      // a learned score without a key or a value: only the denominator knows it
      const float s2 = p.sink[h] * LOG2E, top = fmaxf(m, s2), e = exp2f(m - top);
      f = e / (exp2f(s2 - top) + e * l);
    }
    if (p.gate) f *= hy_sigmoid(p.gate[t * p.ld_gate + h]);
    float* dst = p.out + t * p.ldo + (size_t)h * r + wn * OC + 2 * t4;
#pragma unroll
    for (int j = 0; j < OC / 8; ++j) {
      if (wn * OC + 8 * j < r)
        *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[j][2 * half] * f, o[j][2 * half + 1] * f);
    }
  }
}

template <int RP> int ltc_launch(const LtcParams& p, int tiles, int R, cudaStream_t stream) {
  constexpr int NSPLIT = RP > 256 ? 2 : 1;
  const size_t smem = sizeof(bf16) * 3 * LTC_ROWS * (size_t)p.stride;
  static size_t allowed = 48 * 1024;       // raised once per size, before any stream capture replays the launch
  if (smem > allowed) {
    if (cudaFuncSetAttribute(latent_attention_tc_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return -1;
    allowed = smem;
  }
  gb_launch(latent_attention_tc_kernel<RP>, dim3(tiles, R, p.splits), dim3(128 * NSPLIT), smem, stream, p);
  return 0;
}

// out[t, h, :] = x[t, h, :] W[h]^T on tensor cores, for the two per-head products around the attention (W_uk^T on the
// queries, W_uv on the weighted latents) when a step has rows enough.  A CTA takes 64 rows x 64 outputs of one head
// in steps of 32 inputs; x is 32-bit and rounded to bfloat16 on its way into shared memory, as the framework's other
// products round their inputs; the next step's operands are on their way in registers while this step's multiply.
constexpr int HLT_STRIDE = 40;     // bfloat16 entries a row of a 64 x 32 tile takes (80 bytes: ldmatrix without conflicts)

template <typename TO>
__global__ void __launch_bounds__(128) head_linear_tc_kernel(const float* x, long long ldx, long long xh,
                                                             const bf16* __restrict__ W, TO* out, long long ldo,
                                                             long long oh, int n, int O, int I, const float* gate,
                                                             long long ld_gate) {
  __shared__ __align__(16) bf16 As[64 * HLT_STRIDE];
  __shared__ __align__(16) bf16 Bs[64 * HLT_STRIDE];
  pdl_trigger();
  const int lane = threadIdx.x & 31, wm = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.z, r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const float* xb = x + (size_t)h * xh;
  const bf16* wb = W + (size_t)h * O * I;
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float4 ra[4];
  uint4 rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = threadIdx.x + 128 * u, row = idx >> 3, c = k0 + 4 * (idx & 7);
      ra[u] = (r0 + row < n && c < I) ? *reinterpret_cast<const float4*>(xb + (size_t)(r0 + row) * ldx + c)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int idx = threadIdx.x + 128 * u, row = idx >> 2, c = k0 + 8 * (idx & 3);
      rb[u] = (c0 + row < O && c < I) ? *reinterpret_cast<const uint4*>(wb + (size_t)(c0 + row) * I + c)
                                      : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto put = [&]() {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = threadIdx.x + 128 * u, row = idx >> 3, c = 4 * (idx & 7);
      uint2 w;
      w.x = ltc_pack(ra[u].x, ra[u].y);
      w.y = ltc_pack(ra[u].z, ra[u].w);
      *reinterpret_cast<uint2*>(As + row * HLT_STRIDE + c) = w;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int idx = threadIdx.x + 128 * u, row = idx >> 2, c = 8 * (idx & 3);
      *reinterpret_cast<uint4*>(Bs + row * HLT_STRIDE + c) = rb[u];
    }
  };
  pdl_wait();
  fetch(0);
  for (int k0 = 0; k0 < I; k0 += 32) {
    __syncthreads();                                       // the last step's tiles have been used
    put();
    __syncthreads();
    if (k0 + 32 < I) fetch(k0 + 32);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      unsigned a[4];
      ltc_ldmatrix(a, As + (wm * 16 + (lane & 15)) * HLT_STRIDE + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        unsigned bb[4];
        ltc_ldmatrix(bb, Bs + (np * 16 + (lane & 7) + (lane >> 4) * 8) * HLT_STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
        ltc_mma(acc[2 * np], a, bb[0], bb[1]);
        ltc_mma(acc[2 * np + 1], a, bb[2], bb[3]);
      }
    }
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = r0 + wm * 16 + g + 8 * half;
    if (row >= n) continue;
    TO* dst = out + (size_t)row * ldo + (size_t)h * oh;
    // (a gate logit per output element, laid out like the outputs of a row)
    const float* gt = gate ? gate + (size_t)row * ld_gate + (size_t)h * oh : nullptr;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = c0 + 8 * j + 2 * t4;
      if (col < O) dst[col] = from_f32<TO>(gt ? acc[j][2 * half] * hy_sigmoid(gt[col]) : acc[j][2 * half]);
      if (col + 1 < O) dst[col + 1] = from_f32<TO>(gt ? acc[j][2 * half + 1] * hy_sigmoid(gt[col + 1]) : acc[j][2 * half + 1]);
    }
  }
}

}  // namespace

// Whether the per-head product runs on tensor cores: bfloat16 weights whose rows can be read in 16-byte pieces, 32-bit
// inputs readable four at a time, and at least a tile of rows.
bool gb_head_linear_tc_takes(int n, int I, long long ldx, long long xh, const void* x, const void* W) {
  return n >= 64 && I % 8 == 0 && ldx % 4 == 0 && xh % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

void gb_head_linear_tc_launch(const float* x, long long ldx, long long xh, const bf16* W, void* out, bool out_bf16,
                              long long ldo, long long oh, int n, int H, int O, int I, const float* gate,
                              long long ld_gate, cudaStream_t stream) {
  const dim3 grid(gb_div_up(O, 64), gb_div_up(n, 64), H), block(128);
  if (out_bf16)
    gb_launch(head_linear_tc_kernel<bf16>, grid, block, 0, stream, x, ldx, xh, W, static_cast<bf16*>(out), ldo, oh, n, O, I,
              gate, ld_gate);
  else
    gb_launch(head_linear_tc_kernel<float>, grid, block, 0, stream, x, ldx, xh, W, static_cast<float*>(out), ldo, oh, n, O, I,
              gate, ld_gate);
}

// Whether the tensor-core kernel takes a launch: bfloat16 pages whose rows can be copied in 16-byte pieces (a latent
// and a rotated part of multiples of 8 entries, together at most 576, which is what three tiles of 64 rows leave room
// for in shared memory), no window, at most 64 heads, and a step that carries portions (eight tokens a request on
// average).
bool gb_latent_attention_tc_takes(int n, int R, int H, int r, int dr, int window, bool pages_bf16, const void* pages,
                                  const void* qp, const void* out, long long ldo) {
  return pages_bf16 && dr >= 0 && dr % 8 == 0 && r + dr <= 576 && window == 0 && H >= 1 && H <= LTC_ROWS && r % 8 == 0 && r >= 8 && r <= 512 && R >= 1 &&
         n >= 8 * R && (long long)n * H >= 256 && ((uintptr_t)pages & 15) == 0 && ((uintptr_t)qp & 15) == 0 &&
         ((uintptr_t)out & 7) == 0 && ldo % 2 == 0;
}

// Returns the number of partial results a row has after the launch (1: `out` is final; 2: the caller merges the
// workspace's partial results), or -1 when the kernel's shared memory could not be had.  The key tiles are split in
// two when the launch has few CTAs (a long prompt of one or two requests) and the workspace has the rows.
int gb_latent_attention_tc_launch(const float* qp, const bf16* pages, const int* block_table, int bt_stride, int page_size,
                                  int n_pages, const int* tok_req, const int* tok_pos, const int* q_start,
                                  const float* gate, long long ld_gate, float* out, long long ldo, int n, int R, int H, int r,
                                  int dr, float scale, const float* sink, float* ws, long long ws_rows, int* status,
                                  cudaStream_t stream) {
  LtcParams p;
  p.ws = ws;
  p.dk = r + dr;
  p.stride = 16 * ((p.dk + 15) / 16) + 8;
  p.qp = qp; p.pages = pages; p.block_table = block_table; p.bt_stride = bt_stride; p.page_size = page_size;
  p.n_pages = n_pages; p.tok_req = tok_req; p.tok_pos = tok_pos; p.q_start = q_start; p.n = n; p.R = R; p.gate = gate;
  p.ld_gate = ld_gate; p.out = out; p.ldo = ldo; p.H = H; p.r = r; p.tpt = LTC_ROWS / H;
  p.scale_log2 = scale * 1.4426950408889634f; p.sink = sink; p.status = status;
  const int tiles = gb_div_up(n, p.tpt);                   // (no request has more tokens than the step)
  // (which way a launch goes depends on its numbers of tokens, requests and heads only)
  // two halves where the row tiles alone do not fill the GPU's resident CTAs (two an SM by registers, fewer where three
  // tiles of rows need more than half of an SM's shared memory)
  const size_t smem = sizeof(bf16) * 3 * LTC_ROWS * (size_t)p.stride;
  const int resident = 148 * (smem <= 113 * 1024 ? 2 : 1);
  p.splits = (LTC_SPLIT_KEYS && ws != nullptr && (long long)tiles * R <= resident && n >= 512 * R && 2LL * n * H <= ws_rows) ? 2 : 1;
  int rc;
  if (r <= 64) rc = ltc_launch<64>(p, tiles, R, stream);
  else if (r <= 128) rc = ltc_launch<128>(p, tiles, R, stream);
  else if (r <= 256) rc = ltc_launch<256>(p, tiles, R, stream);
  else rc = ltc_launch<512>(p, tiles, R, stream);
  return rc < 0 ? rc : p.splits;
}
