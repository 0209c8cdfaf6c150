// The attention of gated_attention.cu on the tensor cores, for bfloat16 queries and pages: keys of DK and
// values of DV entries (multiples of 16, which may differ), sliding window, soft cap, sink, output gate.
//
// The rows of a CTA's tile are (token, query head of one kv group) pairs of consecutive tokens of ONE
// request, so the keys and values of a kv head are read from the pages once for all the query heads that
// share them.  A CTA walks the visible keys in tiles of 64 positions (cp.async into two buffers, looked up
// page by page), computes S = Q K^T and O += P V with mma.sync m16n8k16, and keeps scores, soft cap,
// exponentials, maxima and sums in 32-bit.  The weights enter the second product as TWO bfloat16 terms
// (p = hi + lo, O += hi V + lo V), which keeps 16 bits of every weight.  With several chunks of keys
// (blockIdx.z) a CTA leaves (maximum, sum, weighted sum) per row for the merge kernel of gated_attention.cu.
//
// With `maps` > 1 a query head is `maps` heads of DK entries side by side and a key row of the pages holds
// `maps` keys side by side; every map is an attention of its own over the same values with an output of its
// own (differential attention combines them afterwards).  A CTA then takes one (kv head, map) pair.  With
// `blocked` a position sees the positions of its own block of `window` positions, counted from 0, instead
// of the last `window`.  The output is bfloat16 or, for what is combined in 32-bit afterwards, 32-bit.
#include <cuda_bf16.h>

#include "hybrid.cuh"

namespace {

enum { STATUS_BAD_PAGE_READ = 2 };
constexpr int TC_KT = 64, TC_ROWS = 64, TC_THREADS = 128;
static_assert(TC_THREADS == 2 * TC_KT, "two threads copy a key row");

__device__ __forceinline__ void cp16_zfill(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;               // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// the hardware's 2^x and 1/x (a few 2^-23 relative; 2^-inf = 0, 1/inf = 0)
__device__ __forceinline__ float tc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tc_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// p as two bfloat16 terms, packed for two neighbouring columns
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const float2 hf = __bfloat1622float2(h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

struct TcParams {
  const bf16* q; long long ldq;
  const bf16* k_pages; const bf16* v_pages;
  const int* block_table; int bt_stride, page_size, n_pages;
  const int* tok_req; const int* tok_pos; const int* q_start;
  const float* gate; long long ld_gate;
  bf16* out; float* out_f32; long long ldo;      // one of the two
  int N, R, H, G, tokens_per_tile, maps, blocked;
  float scale, softcap;
  int window, sink, splits, chunk;
  const float* sink_scores;      // a learned score of the sink per head, or null: 0
  int keep_first;                // a windowed position also sees the positions below this number
  float* ws; int* status;
};

// Scores are kept times log2(e), so that a weight is one subtraction and one 2^x: with a cap c,
//   c tanh(s / c) log2(e) = c log2(e) - 2 c log2(e) / (2^(s * 2 log2(e) / c) + 1)      (tanh(x) = 1 - 2 / (e^(2x) + 1))
// is a product, a 2^x, a sum, a reciprocal and a multiply-add; without one it is one product.
template <int DK, int DV, bool NARROW>
__global__ void __launch_bounds__(TC_THREADS, (DK + DV <= 128) ? 4 : 2) sink_attention_tc_kernel(TcParams p) {
  constexpr int KS = DK + 8, VS = DV + 8;                    // elements between rows in shared memory
  extern __shared__ __align__(16) unsigned char tc_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(tc_smem);               // [TC_ROWS][KS]
  bf16* Ks = Qs + TC_ROWS * KS;                              // [2][TC_KT][KS]
  bf16* Vs = Ks + 2 * TC_KT * KS;                            // [2][TC_KT][VS]
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = p.H / p.G, tpt = p.tokens_per_tile;
  const int g = blockIdx.y / p.maps, mp = blockIdx.y - g * p.maps;      // kv head and map
  // this CTA's request and first token: the tiles of the step's requests, one request after the other
  int tile = blockIdx.x, t0 = -1, n_tok = 0;
  for (int r = 0; r < p.R; ++r) {
    const int qs = p.q_start[r], qe = r + 1 < p.R ? p.q_start[r + 1] : p.N;
    const int tiles = (qe - qs + tpt - 1) / tpt;
    if (tile < tiles) {
      t0 = qs + tile * tpt;
      n_tok = min(tpt, qe - t0);
      break;
    }
    tile -= tiles;
  }
  if (t0 < 0) return;
  const int pos0 = p.tok_pos[t0];
  const int* table = p.block_table + (size_t)p.tok_req[t0] * p.bt_stride;
  const int n_rows = n_tok * group;
  const int lo = p.window > 0 ? (p.blocked ? (pos0 / p.window) * p.window : max(0, pos0 - p.window + 1)) : 0;
  // the keys the tile may see, in order: the first `kept` positions of the sequence that lie in front of the first
  // token's window, then lo .. the last token's position; key number v of this list is position v (v < kept) or
  // v + shift
  const int kept = (p.window > 0 && !p.blocked) ? min(p.keep_first, lo) : 0;
  const int shift = lo - kept;
  const int k_last = kept + pos0 + n_tok - 1 - lo;
  const int k_begin = p.splits > 1 ? (int)blockIdx.z * p.chunk : 0;
  const int k_end = p.splits > 1 ? min(k_last, k_begin + p.chunk - 1) : k_last;
  const int n_tiles = k_end >= k_begin ? (k_end - k_begin) / TC_KT + 1 : 0;

  // two threads a key row: the row's page is looked up once, each thread copies half of the row's 16-byte pieces
  auto load_kv = [&](int it, int buf) {
    constexpr int PARTS = DK / 8 + DV / 8, HALF = PARTS / 2;
    const int k0 = k_begin + it * TC_KT;
    bf16* kd = Ks + buf * TC_KT * KS;
    bf16* vd = Vs + buf * TC_KT * VS;
    const int j = tid >> 1, first = (tid & 1) * HALF;
    const int kv = k0 + j;
    const int kp = kv < kept ? kv : kv + shift;
    long long row = -1;
    if (kv <= k_end) {
      const int page = table[kp / p.page_size];
      if (page < 0 || page >= p.n_pages) atomicExch(p.status, STATUS_BAD_PAGE_READ);
      else row = ((long long)page * p.G + g) * p.page_size + kp % p.page_size;
    }
    const bf16* ksrc = p.k_pages + ((row < 0 ? 0 : row) * p.maps + mp) * DK;
    const bf16* vsrc = p.v_pages + (row < 0 ? 0 : row) * DV;
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
      const int part = first + i;
      if (part < DK / 8) cp16_zfill(kd + j * KS + part * 8, ksrc + part * 8, row >= 0);
      else cp16_zfill(vd + j * VS + (part - DK / 8) * 8, vsrc + (part - DK / 8) * 8, row >= 0);
    }
    cp_commit();
  };

  pdl_wait();
  // queries of the tile: row R is (token t0 + R / group, head g * group + R % group)
  for (int c = tid; c < TC_ROWS * (DK / 8); c += TC_THREADS) {
    const int R = c / (DK / 8), part = c - R * (DK / 8);
    const bool valid = R < n_rows;
    const int tt = valid ? R / group : 0, hh = valid ? R - tt * group : 0;
    cp16_zfill(Qs + R * KS + part * 8,
               p.q + (size_t)(t0 + tt) * p.ldq + ((size_t)(g * group + hh) * p.maps + mp) * DK + part * 8, valid);
  }
  cp_commit();
  if (n_tiles > 0) load_kv(0, 0);
  cp_wait<0>();
  __syncthreads();

  // NARROW (a tile of up to 16 rows: decoding): the four warps share the rows and split every key tile, warp w
  // taking its keys 16 w .. 16 w + 15; their partial results meet in shared memory at the end
  constexpr int NB = NARROW ? 1 : TC_KT / 16;                // blocks of 16 keys a warp takes of a tile
  const int rb = NARROW ? 0 : warp * 16;                     // the warp's first row
  const bool warp_live = rb < n_rows;
  uint32_t qf[DK / 16][4];
  if (warp_live) {
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk)
      ldsm_x4(qf[kk], Qs + (rb + (lane & 7) + ((lane >> 3) & 1) * 8) * KS + kk * 16 + (lane >> 4) * 8);
  }
  // this thread's two rows and their positions
  const int r_lo = rb + (lane >> 2), r_hi = r_lo + 8;
  const int pos_lo = r_lo < n_rows ? pos0 + r_lo / group : -1, pos_hi = r_hi < n_rows ? pos0 + r_hi / group : -1;
  const int first_lo = p.window <= 0 ? 0 : p.blocked ? (max(pos_lo, 0) / p.window) * p.window : pos_lo - p.window + 1;
  const int first_hi = p.window <= 0 ? 0 : p.blocked ? (max(pos_hi, 0) / p.window) * p.window : pos_hi - p.window + 1;
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  const bool capped = p.softcap > 0.f;
  const float c_in = capped ? p.scale * 2.f * LOG2E / p.softcap : p.scale * LOG2E;
  const float c_mul = -2.f * p.softcap * LOG2E, c_add = p.softcap * LOG2E;
  const int pos_last = pos0 + n_tok - 1;

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) {
      load_kv(it + 1, (it + 1) & 1);
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    if (warp_live) {
      const bf16* kb = Ks + (it & 1) * TC_KT * KS;
      const bf16* vb = Vs + (it & 1) * TC_KT * VS;
      const int k0 = k_begin + it * TC_KT;
      // every row of the tile sees every key of this key tile: nothing to mask
      // (k0 counts visible keys; kr is the position of the tile's first key when the tile lies behind the kept ones)
      const int kr = k0 + shift;
      const bool all_seen = n_rows - rb >= 16 && k0 + TC_KT - 1 <= k_end &&
                            (k0 + TC_KT <= kept ||
                             (k0 >= kept && kr + TC_KT - 1 <= pos0 &&
                              (p.window <= 0 || (p.blocked ? kr >= (pos_last / p.window) * p.window : kr > pos_last - p.window))));
      float s[2 * NB][4];
#pragma unroll
      for (int n = 0; n < 2 * NB; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const int n2 = NARROW ? warp : nb;
          uint32_t b[4];
          ldsm_x4(b, kb + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * KS + kk * 16 + ((lane >> 3) & 1) * 8);
          mma16816(s[2 * nb], qf[kk], b[0], b[1]);
          mma16816(s[2 * nb + 1], qf[kk], b[2], b[3]);
        }
      }
      // scale, soft cap, mask; the rows' maxima
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2 * NB; ++n) {
        const int kcol = k0 + ((NARROW ? 2 * warp : 0) + n) * 8 + (lane & 3) * 2;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * c_in;
          if (capped) v = fmaf(c_mul, tc_rcp(tc_ex2(v) + 1.f), c_add);
          if (!all_seen) {
            const int kv = kcol + (e & 1);
            const int kp = kv < kept ? kv : kv + shift;
            const int pos = e < 2 ? pos_lo : pos_hi, first = e < 2 ? first_lo : first_hi;
            if (kp > pos || (kp < first && kp >= p.keep_first) || kv > k_end) v = -INFINITY;
          }
          s[n][e] = v;
          if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float use_lo = mn_lo == -INFINITY ? 0.f : mn_lo, use_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float c_lo = tc_ex2(m_lo - use_lo), c_hi = tc_ex2(m_hi - use_hi);   // 0 while the row has seen nothing
      m_lo = mn_lo; m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int n = 0; n < 2 * NB; ++n) {
        s[n][0] = tc_ex2(s[n][0] - use_lo); s[n][1] = tc_ex2(s[n][1] - use_lo);
        s[n][2] = tc_ex2(s[n][2] - use_hi); s[n][3] = tc_ex2(s[n][3] - use_hi);
        sum_lo += s[n][0] + s[n][1];
        sum_hi += s[n][2] + s[n][3];
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      l_lo = l_lo * c_lo + sum_lo;
      l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
        o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi;
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const int j = NARROW ? warp : nb;
        uint32_t ph[4], pl[4];
        split2(s[2 * nb][0], s[2 * nb][1], ph[0], pl[0]);
        split2(s[2 * nb][2], s[2 * nb][3], ph[1], pl[1]);
        split2(s[2 * nb + 1][0], s[2 * nb + 1][1], ph[2], pl[2]);
        split2(s[2 * nb + 1][2], s[2 * nb + 1][3], ph[3], pl[3]);
#pragma unroll
        for (int n2 = 0; n2 < DV / 16; ++n2) {
          uint32_t b[4];
          ldsm_x4_t(b, vb + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + n2 * 16 + (lane >> 4) * 8);
          mma16816(o[2 * n2], ph, b[0], b[1]);
          mma16816(o[2 * n2 + 1], ph, b[2], b[3]);
          mma16816(o[2 * n2], pl, b[0], b[1]);
          mma16816(o[2 * n2 + 1], pl, b[2], b[3]);
        }
      }
    }
    __syncthreads();                                         // the buffer is free for the tile after the next
  }

  m_lo *= LN2;                                               // maxima in natural units again (-inf stays)
  m_hi *= LN2;
  if (NARROW) {
    // the warps' partial results, [warp][row][maximum, sum, DV values], over the key buffers (all tiles are used)
    float* part = reinterpret_cast<float*>(Ks);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int R = half ? r_hi : r_lo;
      float* w = part + ((size_t)warp * 16 + R) * (DV + 2);
      if ((lane & 3) == 0) { w[0] = half ? m_hi : m_lo; w[1] = half ? l_hi : l_lo; }
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
        w[2 + n * 8 + (lane & 3) * 2] = o[n][2 * half];
        w[2 + n * 8 + (lane & 3) * 2 + 1] = o[n][2 * half + 1];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < n_rows * DV; idx += TC_THREADS) {
      const int R = idx / DV, d = idx - R * DV;
      const int tt = R / group, h = (g * group + (R - tt * group)) * p.maps + mp, t = t0 + tt;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) m = fmaxf(m, part[((size_t)w * 16 + R) * (DV + 2)]);
      float l = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {                           // in warp order
        const float* pw = part + ((size_t)w * 16 + R) * (DV + 2);
        if (pw[0] > -INFINITY) {
          const float e = expf(pw[0] - m);
          l = fmaf(e, pw[1], l);
          acc = fmaf(e, pw[2 + d], acc);
        }
      }
      if (p.splits > 1) {
        float* w = p.ws + (((size_t)t * p.H * p.maps + h) * p.splits + blockIdx.z) * (DV + 2);
        if (d == 0) { w[0] = m; w[1] = l; }
        w[2 + d] = acc;
        continue;
      }
      const float z = p.sink_scores ? p.sink_scores[h / p.maps] : 0.f;
      const float M = p.sink ? fmaxf(m, z) : m;
      const float e = expf(m - M);
      const float inv = 1.0f / fmaf(e, l, p.sink ? expf(z - M) : 0.f);
      const float gt = p.gate ? hy_sigmoid(p.gate[(size_t)t * p.ld_gate + (size_t)h * DV + d]) : 1.f;
      const float val = fmaf(e, acc, 0.f) * inv * gt;
      if (p.out_f32) p.out_f32[(size_t)t * p.ldo + (size_t)h * DV + d] = val;
      else p.out[(size_t)t * p.ldo + (size_t)h * DV + d] = __float2bfloat16_rn(val);
    }
    return;
  }
  if (!warp_live) return;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int R = half ? r_hi : r_lo;
    if (R >= n_rows) continue;
    const int tt = R / group, h = (g * group + (R - tt * group)) * p.maps + mp, t = t0 + tt;
    const float m = half ? m_hi : m_lo, l = half ? l_hi : l_lo;
    if (p.splits > 1) {
      float* w = p.ws + (((size_t)t * p.H * p.maps + h) * p.splits + blockIdx.z) * (DV + 2);
      if ((lane & 3) == 0) { w[0] = m; w[1] = l; }
#pragma unroll
      for (int n = 0; n < DV / 8; ++n) {
        w[2 + n * 8 + (lane & 3) * 2] = o[n][2 * half];
        w[2 + n * 8 + (lane & 3) * 2 + 1] = o[n][2 * half + 1];
      }
      continue;
    }
    // (the same arithmetic as the merge of chunks: one chunk, and the sink)
    const float z = p.sink_scores ? p.sink_scores[h / p.maps] : 0.f;
    const float M = p.sink ? fmaxf(m, z) : m;
    const float e = expf(m - M);
    const float inv = 1.0f / fmaf(e, l, p.sink ? expf(z - M) : 0.f);
    const float* gt = p.gate ? p.gate + (size_t)t * p.ld_gate + (size_t)h * DV : nullptr;
    const size_t at = (size_t)t * p.ldo + (size_t)h * DV;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      const int d = n * 8 + (lane & 3) * 2;
      const float g0 = gt ? hy_sigmoid(gt[d]) : 1.f, g1 = gt ? hy_sigmoid(gt[d + 1]) : 1.f;
      const float v0 = fmaf(e, o[n][2 * half], 0.f) * inv * g0, v1 = fmaf(e, o[n][2 * half + 1], 0.f) * inv * g1;
      if (p.out_f32) *reinterpret_cast<float2*>(p.out_f32 + at + d) = make_float2(v0, v1);
      else *reinterpret_cast<__nv_bfloat162*>(p.out + at + d) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

template <int DK, int DV, bool NARROW>
int launch_tc(const TcParams& p, dim3 grid, cudaStream_t stream) {
  constexpr int smem = (TC_ROWS * (DK + 8) + 2 * TC_KT * (DK + 8) + 2 * TC_KT * (DV + 8)) * 2;
  static bool raised = false;            // once per size, before any stream capture replays the launch
  if (!raised && smem > 48 * 1024) {
    GB_CUDA((cudaFuncSetAttribute(sink_attention_tc_kernel<DK, DV, NARROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)));
    raised = true;
  }
  gb_launch(sink_attention_tc_kernel<DK, DV, NARROW>, grid, dim3(TC_THREADS), smem, stream, p);
  GB_CHECK_LAUNCH("sink_attention_tc");
  return 1;
}

}  // namespace

// (gated_attention.cu)
int gb_sink_attention_merge(const float* ws, int splits, const float* gate, long long ld_gate, void* out, int out_bf16,
                            long long ldo, int n, int H, int vdim, int sink, const float* sink_scores, int maps,
                            cudaStream_t stream);
extern "C" int gb_sink_attention_workspace_rows();

// Whether the tensor-core kernel takes these sizes (keys and values of 32 to 128 entries in steps of 32, up to
// 64 query heads a kv head, rows that 16-byte copies can address).
GB_API int gb_sink_attention_tc_supported(int heads, int kv_heads, int dim, int vdim) {
  if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > TC_ROWS) return 0;
  const bool dk = dim == 32 || dim == 64 || dim == 96 || dim == 128;
  const bool dv = vdim == 32 || vdim == 64 || vdim == 96 || vdim == 128;
  return dk && dv;
}

// a0 q [tokens, heads * dim] (bf16), a1 key pages, a2 value pages (bf16), a3 block table, a4 its entries per request,
// a5 page size, a6 number of pages, a7 token -> request, a8 token -> position, a9 gate logits (f32) or 0, a10 their row
// stride, a11 out [tokens, heads * vdim] (bf16), a12 its row stride, a13 tokens, a14 heads, a15 kv heads, a16 dim,
// a17 vdim, a18 window (0: every earlier position), a19 longest context of the step (an upper bound will do), a20
// workspace for partial results (gb_sink_attention_workspace_rows() rows of vdim + 2 floats) or 0, a21 requests, a22
// row of each request's first token [requests]; flags bit 0: the softmax has a sink, bit 1: out is 32-bit (else
// bfloat16), bit 2: a position sees its own block of `window` positions, counted from 0, bits 8 to 11: maps (0 means
// 1): q is [tokens, heads * maps * dim], a key row [maps * dim], out [tokens, heads * maps * vdim]; a23 a learned score
// of the sink per head (f32 [heads]) or 0: the sink's score is 0; f0 scale, f1 soft cap (0: none), f2 keep_first: a
// windowed position also sees the positions below this number
GB_OP(gb_op_sink_attention_tc) {
  const int n = (int)a[13], H = (int)a[14], G = (int)a[15], dim = (int)a[16], vdim = (int)a[17], R = (int)a[21];
  if (n <= 0 || R <= 0) return 0;
  if (!gb_sink_attention_tc_supported(H, G, dim, vdim))
    GB_FAIL(GB_ERR_ARG, "sink_attention_tc: %d heads over %d kv heads of %d / %d entries are not built", H, G, dim, vdim);
  const int maps = ((flags >> 8) & 15) ? ((flags >> 8) & 15) : 1;
  const bool out_f32 = flags & 2;
  if ((a[0] & 15) || (a[1] & 15) || (a[2] & 15) || (a[11] & (out_f32 ? 7 : 3)) || (a[12] & 1))
    GB_FAIL(GB_ERR_ARG, "sink_attention_tc: operands are not aligned for 16-byte copies");
  if ((flags & 4) && a[18] <= 0) GB_FAIL(GB_ERR_ARG, "sink_attention_tc: blocks of %lld positions", a[18]);
  if (maps > 1 && a[9]) GB_FAIL(GB_ERR_ARG, "sink_attention_tc: no output gate with several maps");
  const int group = H / G;
  TcParams p;
  p.maps = maps; p.blocked = (flags & 4) ? 1 : 0;
  p.q = op_ptr<const bf16>(a[0]); p.ldq = (long long)H * maps * dim;
  p.k_pages = op_ptr<const bf16>(a[1]); p.v_pages = op_ptr<const bf16>(a[2]);
  p.block_table = op_ptr<const int>(a[3]); p.bt_stride = (int)a[4]; p.page_size = (int)a[5]; p.n_pages = (int)a[6];
  p.tok_req = op_ptr<const int>(a[7]); p.tok_pos = op_ptr<const int>(a[8]); p.q_start = op_ptr<const int>(a[22]);
  p.gate = op_ptr<const float>(a[9]); p.ld_gate = a[10];
  p.out = out_f32 ? nullptr : op_ptr<bf16>(a[11]); p.out_f32 = out_f32 ? op_ptr<float>(a[11]) : nullptr; p.ldo = a[12];
  // every request brings one token (n == R) and its heads fill at most 16 rows: tiles of one token, whose key tiles
  // the four warps split
  const bool narrow = n == R && group <= 16;
  p.N = n; p.R = R; p.H = H; p.G = G; p.tokens_per_tile = narrow ? 1 : TC_ROWS / group;
  p.scale = (float)f[0]; p.softcap = (float)f[1];
  p.window = (int)a[18]; p.sink = flags & 1;
  p.sink_scores = op_ptr<const float>(a[23]);
  p.keep_first = (p.window > 0 && !p.blocked) ? (int)f[2] : 0;
  if (p.keep_first < 0) GB_FAIL(GB_ERR_ARG, "sink_attention_tc: %d kept first positions", p.keep_first);
  if (p.sink_scores && !p.sink) GB_FAIL(GB_ERR_ARG, "sink_attention_tc: learned sink scores without a sink");
  p.ws = op_ptr<float>(a[20]); p.status = ctx->status;
  // at most this many tiles: every request may end with a partial one
  const int tiles = narrow ? n : gb_div_up(n, p.tokens_per_tile) + R;
  // chunks of keys when the tiles alone leave the GPU idle (decoding); whole key tiles, at fixed distances from the
  // first visible key; with a window the cut depends on the launch's sizes only
  const int span = p.window > 0 ? p.window + p.keep_first + p.tokens_per_tile : (a[19] > 0 ? (int)a[19] : 1);
  int wanted = 592 / (tiles * G * maps);
  if (wanted > 32) wanted = 32;
  p.splits = 1; p.chunk = span;
  if (wanted > 1 && p.ws != nullptr && !(p.window > 0 && span <= TC_KT)) {
    int chunk;
    if (p.window > 0) {
      chunk = TC_KT * gb_div_up(gb_div_up(span, wanted), TC_KT);
    } else {
      chunk = 256;
      while (gb_div_up(span, chunk) > 2 * wanted) chunk *= 2;
    }
    const int splits = gb_div_up(span, chunk);
    if (splits > 1 && (long long)n * H * maps * splits <= gb_sink_attention_workspace_rows()) {
      p.splits = splits;
      p.chunk = chunk;
    }
  }
  const dim3 grid(tiles, G * maps, p.splits);
  int rc;
#define TC(DK, DV) rc = narrow ? launch_tc<DK, DV, true>(p, grid, ctx->stream) : launch_tc<DK, DV, false>(p, grid, ctx->stream)
#define TC_DV(DK)                                                                                    \
  do {                                                                                               \
    if (vdim == 32) TC(DK, 32); else if (vdim == 64) TC(DK, 64); else if (vdim == 96) TC(DK, 96); else TC(DK, 128); \
  } while (0)
  if (dim == 32) TC_DV(32); else if (dim == 64) TC_DV(64); else if (dim == 96) TC_DV(96); else TC_DV(128);
#undef TC_DV
#undef TC
  if (rc < 0) return rc;
  if (p.splits == 1) return 1;
  rc = gb_sink_attention_merge(p.ws, p.splits, p.gate, p.ld_gate, out_f32 ? (void*)p.out_f32 : (void*)p.out, out_f32 ? 0 : 1,
                               p.ldo, n, H * maps, vdim, p.sink, p.sink_scores, maps, ctx->stream);
  return rc < 0 ? rc : 2;
}
