// Attention over a compressed ("latent") key/value cache, in the absorbed form.
//
// A token's cache row is [c | k_rot]: the RMS-normed latent c (kv_rank values), from which every head's
// unrotated keys W_uk c and values W_uv c derive, and one rotated key part shared by all heads.  With
//   q'_h = [W_uk,h^T q_plain,h | rot(q_rot,h)]
// the score of head h against a cached row is q'_h . [c | k_rot], and the head's output is
// W_uv,h (sum_j p_j c_j): nothing but the cache rows is read per key, for prompts and decoding alike.
//
//  gb_op_latent_prep       RMS norm of the latent and rotation of the shared key part, written into the
//                          token's page; rotation of the queries' rotated parts into q'
//  gb_op_head_linear       out[t, h, :] = x[t, h, :] W[h]^T for every head (absorbing W_uk, applying W_uv)
//  gb_op_latent_attention  softmax(scale * q' . rows) over the last `window` rows (all when 0), times the
//                          rows' latent part, times sigmoid(gate[t, h]) where there is a gate; with a sink,
//                          exp(sink[h]) is added to the softmax's denominator; scores and weights in 32-bit
//
// Rotation: the first `rot_dims` entries of a rotated part turn in adjacent pairs (2i, 2i+1) by
// pos * inv_freq[i] (angle in 32-bit); the rest passes unchanged.
// Pages: [n_pages, page_size, kv_rank + rot_dim]; a page id outside the pool is never dereferenced: the
// access is skipped and *status is set.
#include "hybrid.cuh"

namespace {

enum { STATUS_BAD_PAGE_WRITE = 1, STATUS_BAD_PAGE_READ = 2 };

// one block per token: warp 0 writes the cache row, the others rotate the heads' queries
template <typename TC>
__global__ void latent_prep_kernel(const float* fused, long long ld, int dkv_col, const float* queries, long long ldq,
                                   const float* __restrict__ gain,
                                   const float* __restrict__ inv_freq, int rot_dims, const int* tok_req,
                                   const int* tok_pos, const int* block_table, int bt_stride, int page_size, TC* pages,
                                   int n_pages, int H, int dn, int dr, int r, float* qp, float eps, int* status) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pos = tok_pos[t];
  const int half = rot_dims >> 1;
  pdl_wait();
  const float* row = fused + (size_t)t * ld;
  if (warp == 0) {
    const int page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
    if (page < 0 || page >= n_pages) {
      if (lane == 0) atomicExch(status, STATUS_BAD_PAGE_WRITE);
    } else {
      TC* dst = pages + ((size_t)page * page_size + pos % page_size) * (r + dr);
      const float* lat = row + dkv_col;
      float ss = 0.f;
      for (int d = lane; d < r; d += 32) ss += lat[d] * lat[d];
      const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)r + eps);
      for (int d = lane; d < r; d += 32) dst[d] = from_f32<TC>(lat[d] * rstd * gain[d]);
      const float* kr = lat + r;
      for (int j = lane; j < half; j += 32) {
        const float ang = (float)pos * inv_freq[j];
        const float c = cosf(ang), s = sinf(ang);
        const float u = kr[2 * j], v = kr[2 * j + 1];
        dst[r + 2 * j] = from_f32<TC>(u * c - v * s);
        dst[r + 2 * j + 1] = from_f32<TC>(v * c + u * s);
      }
      for (int d = 2 * half + lane; d < dr; d += 32) dst[r + d] = from_f32<TC>(kr[d]);
    }
  }
  const int w0 = warps > 1 ? 1 : 0, step = warps > 1 ? warps - 1 : 1;
  if (warps > 1 && warp == 0) return;
  for (int h = warp - w0; h < H; h += step) {
    const float* q = queries + (size_t)t * ldq + (size_t)h * (dn + dr) + dn;
    float* o = qp + ((size_t)t * H + h) * (r + dr) + r;
    for (int j = lane; j < half; j += 32) {
      const float ang = (float)pos * inv_freq[j];
      const float c = cosf(ang), s = sinf(ang);
      const float u = q[2 * j], v = q[2 * j + 1];
      o[2 * j] = u * c - v * s;
      o[2 * j + 1] = v * c + u * s;
    }
    for (int d = 2 * half + lane; d < dr; d += 32) o[d] = q[d];
  }
}

template <typename TW, typename TO>
__global__ void head_linear_kernel(const float* x, long long ldx, long long xh, const TW* __restrict__ W, TO* out,
                                   long long ldo, long long oh, int n, int O, int I, const float* gate, long long ld_gate) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.z, r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const float* xb = x + (size_t)h * xh;
  const TW* wb = W + (size_t)h * O * I;
  float acc[4][4];
  int ty, tx;
  hy_tile_64x64<float, TW>(
      [&](int i) -> const float* { return r0 + i < n ? xb + (size_t)(r0 + i) * ldx : nullptr; },
      [&](int j) -> const TW* { return c0 + j < O ? wb + (size_t)(c0 + j) * I : nullptr; }, I, acc, ty, tx);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = r0 + ty * 4 + r;
    if (row >= n) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = c0 + tx * 4 + c;
      if (col < O) {
        const float gt = gate ? hy_sigmoid(gate[(size_t)row * ld_gate + (size_t)h * oh + col]) : 1.f;
        out[(size_t)row * ldo + (size_t)h * oh + col] = from_f32<TO>(gate ? acc[r][c] * gt : acc[r][c]);
      }
    }
  }
}

// A few rows (decoding): one block per (8 outputs, head), the head's inputs of all rows in shared memory,
// one warp per output with the lanes over the inputs.
constexpr int HL_SMALL_ROWS = 16;

template <typename TW, typename TO>
__global__ void head_linear_small_kernel(const float* x, long long ldx, long long xh, const TW* __restrict__ W, TO* out,
                                         long long ldo, long long oh, int n, int O, int I, const float* gate,
                                         long long ld_gate) {
  extern __shared__ float xs[];                          // [n][I]
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < n * I; i += blockDim.x) {
    const int t = i / I;
    xs[i] = x[(size_t)t * ldx + (size_t)h * xh + (i - t * I)];
  }
  __syncthreads();
  {
    const int o = blockIdx.x * (blockDim.x >> 5) + warp;
    if (o >= O) return;
    const TW* w = W + ((size_t)h * O + o) * I;
    float acc[HL_SMALL_ROWS];
#pragma unroll
    for (int t = 0; t < HL_SMALL_ROWS; ++t) acc[t] = 0.f;
    for (int i = lane; i < I; i += 32) {
      const float wv = to_f32(w[i]);
#pragma unroll
      for (int t = 0; t < HL_SMALL_ROWS; ++t)
        if (t < n) acc[t] = fmaf(xs[t * I + i], wv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < HL_SMALL_ROWS; ++t) {
      if (t < n) {
        const float v = warp_sum(acc[t]);
        if (lane == 0) {
          const float gt = gate ? hy_sigmoid(gate[(size_t)t * ld_gate + (size_t)h * oh + o]) : 1.f;
          out[(size_t)t * ldo + (size_t)h * oh + o] = from_f32<TO>(gate ? v * gt : v);
        }
      }
    }
  }
}

// A cache row into shared memory as 32-bit values, 16 bytes at a time; `sub` of eight threads share the row.
__device__ __forceinline__ void load_row_vec(const bf16* src, float* dst, int Dk, int sub) {
  // (up to four pieces are requested before any is stored: a store to shared memory in between would make
  // every load wait for the one before it)
  for (int d0 = sub * 8; d0 < Dk; d0 += 256) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (d0 + 64 * u < Dk) raw[u] = *reinterpret_cast<const uint4*>(src + d0 + 64 * u);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int d = d0 + 64 * u;
      if (d < Dk) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f2 = __bfloat1622float2(h2[e]);
          dst[d + 2 * e] = f2.x;
          dst[d + 2 * e + 1] = f2.y;
        }
      }
    }
  }
}
__device__ __forceinline__ void load_row_vec(const float* src, float* dst, int Dk, int sub) {
  for (int d = sub * 4; d < Dk; d += 32) {
    const float4 v = *reinterpret_cast<const float4*>(src + d);
    dst[d] = v.x; dst[d + 1] = v.y; dst[d + 2] = v.z; dst[d + 3] = v.w;
  }
}

// One block per (token, group of up to LA_HB heads, chunk of keys); a warp looks after LA_HW heads, whose
// queries it holds in registers, the lanes over the dimensions of a cache row.  Key rows arrive in tiles
// of LA_KT in shared memory (32-bit), shared by the block's heads.  Per key a warp reads the row ONCE
// (conflict-free, consecutive lanes consecutive values): the same registers give the scores of its heads
// (a product summed over the lanes) and then enter the weighted sums; the softmax is kept per key (the
// sums are rescaled only when a score exceeds the running maximum, a branch the whole warp takes together).
// (Measured against a variant that takes a tile's scores first, lane j keeping key j's, and then the
// weighted sums in a second pass over the tile: 17.9 against 26.0 ms for four layers of a 2,048-token
// prompt at 16 heads, latent 512 + 64, window 1,024.)
// Exponentials of the softmax: the accurate one where the cache is 32-bit; where the cache rows are bfloat16
// (2^-9 relative) the hardware's 2^x, whose error of a few 2^-23 relative is far below what the rows carry.
template <typename TC> __device__ __forceinline__ float la_exp(float x) { return expf(x); }
template <> __device__ __forceinline__ float la_exp<bf16>(float x) { return __expf(x); }

constexpr int LA_HW = 2, LA_WARPS = 8, LA_HB = LA_HW * LA_WARPS, LA_KT = 32, LA_RR = 4;   // rotated part: up to 128

template <typename TC, int RL>
__global__ void __launch_bounds__(32 * LA_WARPS, 2)      // (two blocks an SM: at most 128 registers a thread)
latent_attention_kernel(const float* qp, const TC* pages, const int* block_table, int bt_stride, int page_size,
                        int n_pages, const int* tok_req, const int* tok_pos, const float* gate, long long ld_gate,
                        float* out, long long ldo, int H, int r, int dr, float scale, int window, int splits, int chunk,
                        float* ws, const float* __restrict__ sink, int* status) {
  extern __shared__ __align__(16) float ks[];      // [LA_KT][Dk]
  pdl_trigger();
  const int Dk = r + dr;
  const int t = blockIdx.x, h0 = blockIdx.y * LA_HB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hw = h0 + warp * LA_HW;                // this warp's first head
  const int pos = tok_pos[t];
  const int* table = block_table + (size_t)tok_req[t] * bt_stride;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // rows of pages can be read in 16-byte pieces when their length allows (pages are 16-byte aligned)
  const bool vec = (Dk * (int)sizeof(TC)) % 16 == 0 && (((uintptr_t)pages) & 15) == 0;
  // this block's share of the visible keys lo .. pos: chunk number blockIdx.z, counted from lo
  const int k_begin = splits > 1 ? lo + (int)blockIdx.z * chunk : lo;
  const int k_end = splits > 1 ? min(pos, k_begin + chunk - 1) : pos;
  pdl_wait();
  float ql[LA_HW][RL], qr[LA_HW][LA_RR], acc[LA_HW][RL], m[LA_HW], l[LA_HW];
#pragma unroll
  for (int hh = 0; hh < LA_HW; ++hh) {
    const bool live = hw + hh < H;
    const float* src = qp + ((size_t)t * H + (live ? hw + hh : 0)) * Dk;
#pragma unroll
    for (int i = 0; i < RL; ++i) {
      const int d = lane + 32 * i;
      ql[hh][i] = (live && d < r) ? src[d] : 0.f;
      acc[hh][i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < LA_RR; ++i) {
      const int d = lane + 32 * i;
      qr[hh][i] = (live && d < dr) ? src[r + d] : 0.f;
    }
    m[hh] = -INFINITY;
    l[hh] = 0.f;
  }
  for (int k0 = k_begin; k0 <= k_end; k0 += LA_KT) {
    __syncthreads();                       // the last tile has been used
    {
      // eight threads share a key row; its page is looked up once
      const int sub = threadIdx.x & 7;
      for (int j = threadIdx.x >> 3; j < LA_KT; j += blockDim.x >> 3) {
      const int kp = k0 + j;
      const TC* src = nullptr;
      if (kp <= k_end) {
        const int page = table[kp / page_size];
        if (page < 0 || page >= n_pages) {
          if (sub == 0) atomicExch(status, STATUS_BAD_PAGE_READ);
        } else {
          src = pages + ((size_t)page * page_size + kp % page_size) * Dk;
        }
      }
      float* dst = ks + j * Dk;
      if (src == nullptr) {
        for (int d = sub; d < Dk; d += 8) dst[d] = 0.f;
      } else if (vec) {
        load_row_vec(src, dst, Dk, sub);
      } else {
        for (int d = sub; d < Dk; d += 8) dst[d] = to_f32(src[d]);
      }
      }
    }
    __syncthreads();
    if (hw >= H) continue;
    const int n_keys = min(LA_KT, k_end - k0 + 1);
    // Keys are taken KG at a time: their rows are read and their scores' partial products and warp sums are worked
    // out side by side (independent chains that hide one another's latencies: a step of a few tokens is bound by
    // them), then the softmax takes the keys one after the other.  Every number is computed by the same operations
    // in the same order as with one key at a time.
    constexpr int KG = RL <= 8 ? 4 : 1;                     // (latents beyond 256 entries fill the registers: one key at a time)
    for (int j0 = 0; j0 < n_keys; j0 += KG) {
      float kl[KG][RL], kr[KG][LA_RR], sc[KG][LA_HW];
#pragma unroll
      for (int u = 0; u < KG; ++u) {
        const float* row = ks + min(j0 + u, n_keys - 1) * Dk;      // (a key beyond the tile's last: read again, not used)
#pragma unroll
        for (int i = 0; i < RL; ++i) {
          const int d = lane + 32 * i;
          kl[u][i] = d < r ? row[d] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < LA_RR; ++i) {
          const int d = lane + 32 * i;
          kr[u][i] = d < dr ? row[r + d] : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < KG; ++u) {
#pragma unroll
        for (int hh = 0; hh < LA_HW; ++hh) {
          float p0 = 0.f, p1 = 0.f;                          // two chains; added in a fixed order
#pragma unroll
          for (int i = 0; i < RL; ++i) {
            if (i & 1) p1 = fmaf(ql[hh][i], kl[u][i], p1);
            else p0 = fmaf(ql[hh][i], kl[u][i], p0);
          }
#pragma unroll
          for (int i = 0; i < LA_RR; ++i) {
            if (i & 1) p1 = fmaf(qr[hh][i], kr[u][i], p1);
            else p0 = fmaf(qr[hh][i], kr[u][i], p0);
          }
          sc[u][hh] = p0 + p1;
        }
      }
      // the warp sums of all scores, step by step (every lane gets the same sums)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < KG; ++u) {
#pragma unroll
          for (int hh = 0; hh < LA_HW; ++hh) sc[u][hh] += __shfl_xor_sync(0xffffffffu, sc[u][hh], o);
        }
      }
#pragma unroll
      for (int u = 0; u < KG; ++u) {
        if (j0 + u >= n_keys) break;                         // (the whole warp together)
#pragma unroll
        for (int hh = 0; hh < LA_HW; ++hh) {
          const float s1 = sc[u][hh] * scale;
          if (s1 > m[hh]) {                                  // (the whole warp together)
            const float corr = la_exp<TC>(m[hh] - s1);       // 0 for the first key: m = -inf
            l[hh] *= corr;
#pragma unroll
            for (int i = 0; i < RL; ++i) acc[hh][i] *= corr;
            m[hh] = s1;
          }
          const float p = la_exp<TC>(s1 - m[hh]);
          l[hh] += p;
#pragma unroll
          for (int i = 0; i < RL; ++i) acc[hh][i] = fmaf(p, kl[u][i], acc[hh][i]);
        }
      }
    }
  }
#pragma unroll
  for (int hh = 0; hh < LA_HW; ++hh) {
    const int h = hw + hh;
    if (h >= H) continue;
    if (splits > 1) {
      // partial result of this chunk: running maximum, sum of weights, weighted sum (not yet divided)
      float* w = ws + (((size_t)t * H + h) * splits + blockIdx.z) * (r + 2);
      if (lane == 0) { w[0] = m[hh]; w[1] = l[hh]; }
#pragma unroll
      for (int i = 0; i < RL; ++i) {
        const int d = lane + 32 * i;
        if (d < r) w[2 + d] = acc[hh][i];
      }
      continue;
    }
    const float g = gate ? hy_sigmoid(gate[(size_t)t * ld_gate + h]) : 1.f;
    float inv = g / l[hh], e = 1.f;
    if (sink) {
      // a learned score without a key or a value: it only joins the denominator (by the merge kernel's
      // arithmetic, so that one chunk and several of which one holds keys give the same bits)
      const float top = fmaxf(m[hh], sink[h]);
      e = expf(m[hh] - top);
      inv = g / __fadd_rn(expf(sink[h] - top), __fmul_rn(e, l[hh]));
    }
    float* o = out + (size_t)t * ldo + (size_t)h * r;
#pragma unroll
    for (int i = 0; i < RL; ++i) {
      const int d = lane + 32 * i;
      if (d < r) o[d] = __fmul_rn(e, acc[hh][i]) * inv;
    }
  }
}

// One warp per (token, head): the chunks' partial results, merged in chunk order.
__global__ void latent_attention_merge_kernel(const float* ws, int splits, const float* gate, long long ld_gate,
                                              float* out, long long ldo, int n, int H, int r,
                                              const float* __restrict__ sink) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= (long long)n * H) return;
  const int t = (int)(idx / H), h = (int)(idx - (long long)t * H);
  const float* w = ws + (size_t)idx * splits * (r + 2);
  // the chunks' weights exp(m_s - M) once (lane s for chunk s, 32 chunks at a time), then the columns
  float M = -INFINITY;
  for (int s = lane; s < splits; s += 32) M = fmaxf(M, w[(size_t)s * (r + 2)]);
  M = warp_max(M);
  if (sink) M = fmaxf(M, sink[h]);
  float L = sink ? expf(sink[h] - M) : 0.f;
  for (int s0 = 0; s0 < splits; s0 += 32) {                // in chunk order
    const int s = s0 + lane;
    const float m = s < splits ? w[(size_t)s * (r + 2)] : -INFINITY;
    const float e = m > -INFINITY ? expf(m - M) : 0.f;
    const float el = s < splits ? e * w[(size_t)s * (r + 2) + 1] : 0.f;
    for (int u = 0; u < 32 && s0 + u < splits; ++u) L += __shfl_sync(0xffffffffu, el, u);
  }
  const float g = gate ? hy_sigmoid(gate[(size_t)t * ld_gate + h]) : 1.f;
  const float inv = g / L;
  for (int d0 = 0; d0 < r; d0 += 128) {                    // four columns per lane at a time
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = 0; s0 < splits; s0 += 32) {
      const int s = s0 + lane;
      const float m = s < splits ? w[(size_t)s * (r + 2)] : -INFINITY;
      const float e = m > -INFINITY ? expf(m - M) : 0.f;
      for (int u = 0; u < 32 && s0 + u < splits; ++u) {
        const float eu = __shfl_sync(0xffffffffu, e, u);
        if (eu == 0.f) continue;                             // a chunk without keys (the whole warp together)
        const float* wu = w + (size_t)(s0 + u) * (r + 2) + 2;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int d = d0 + lane + 32 * v;
          if (d < r) a[v] = fmaf(eu, wu[d], a[v]);
        }
      }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int d = d0 + lane + 32 * v;
      if (d < r) out[(size_t)t * ldo + (size_t)h * r + d] = a[v] * inv;
    }
  }
}

}  // namespace

bool gb_head_linear_tc_takes(int n, int I, long long ldx, long long xh, const void* x, const void* W);
void gb_head_linear_tc_launch(const float* x, long long ldx, long long xh, const bf16* W, void* out, bool out_bf16,
                              long long ldo, long long oh, int n, int H, int O, int I, const float* gate, long long ld_gate,
                              cudaStream_t stream);
bool gb_latent_attention_tc_takes(int n, int R, int H, int r, int dr, int window, bool pages_bf16, const void* pages,
                                  const void* qp, const void* out, long long ldo);
int gb_latent_attention_tc_launch(const float* qp, const bf16* pages, const int* block_table, int bt_stride, int page_size,
                                  int n_pages, const int* tok_req, const int* tok_pos, const int* q_start,
                                  const float* gate, long long ld_gate, float* out, long long ldo, int n, int R, int H, int r,
                                  int dr, float scale, const float* sink, float* ws, long long ws_rows, int* status,
                                  cudaStream_t stream);

// How the visible keys of a launch are cut into chunks of whole key tiles: (chunks, keys per chunk).
// Few tokens (decoding) get many chunks, so that the GPU is occupied; a launch with enough (token, head
// group) blocks of its own gets one.  With a window the chunk depends on the launch's sizes only, not on
// the contexts' lengths; chunks lie at fixed distances from the first visible key, so a chunk's partial
// result does not depend on how many chunks there are.
GB_API int gb_latent_attention_chunks(int n, int H, int window, int max_ctx, int* chunk_out) {
  const int blocks = n * gb_div_up(H, LA_HB);
  int wanted = 592 / (blocks > 0 ? blocks : 1);
  if (wanted > 64) wanted = 64;
  const int span = window > 0 ? window : (max_ctx > 0 ? max_ctx : 1);
  if (wanted <= 1 || span <= 32) { *chunk_out = span; return 1; }
  int chunk;
  if (window > 0) {
    chunk = 32 * gb_div_up(gb_div_up(span, wanted), 32);
    if (chunk < 32) chunk = 32;
  } else {
    chunk = 2 * LA_KT;
    while (gb_div_up(span, chunk) > wanted) chunk *= 2;
  }
  *chunk_out = chunk;
  return gb_div_up(span, chunk);
}
// Rows of (latent size + 2) floats a launch's partial results may need, whatever its sizes.
// (also: two partial results a row for a prompt of up to 2,048 tokens and 16 heads on the tensor-core kernel)
GB_API int gb_latent_attention_workspace_rows() { return 65536 > LA_HB * 2 * (592 + 592) ? 65536 : LA_HB * 2 * (592 + 592); }

// a0 fused rows [q heads (plain | rotated) | ... ] (f32), a1 their stride, a2 column of [latent | rotated key],
// a3 gain of the latent's norm [r], a4 inv_freq [rot_dims / 2], a5 rot_dims, a6 token -> request, a7 token ->
// position, a8 block table, a9 its entries per request, a10 page size, a11 pages, a12 number of pages, a13 their dtype,
// a14 tokens, a15 heads, a16 plain query size, a17 rotated size, a18 latent size, a19 q' [tokens, heads, r + rot]
// (f32), a20 the queries [tokens, heads * (plain + rotated)] (f32) when they are no part of the fused rows (they came
// through a product of their own), else 0, a21 their row stride; f0 eps
GB_OP(gb_op_latent_prep) {
  const int n = (int)a[14], H = (int)a[15];
  if (n <= 0) return 0;
  if (a[5] % 2 || a[5] > a[17]) GB_FAIL(GB_ERR_ARG, "latent_prep: %lld rotated dimensions of %lld", a[5], a[17]);
  const int warps = H + 1 < 8 ? H + 1 : 8;
#define PREP(TC)                                                                                                       \
  gb_launch(latent_prep_kernel<TC>, dim3(n), dim3(32 * warps), 0, ctx->stream, op_ptr<const float>(a[0]), a[1], (int)a[2], \
            a[20] ? op_ptr<const float>(a[20]) : op_ptr<const float>(a[0]), a[20] ? a[21] : a[1], op_ptr<const float>(a[3]), \
            op_ptr<const float>(a[4]), (int)a[5], op_ptr<const int>(a[6]),                   \
            op_ptr<const int>(a[7]), op_ptr<const int>(a[8]), (int)a[9], (int)a[10], op_ptr<TC>(a[11]), (int)a[12], H,  \
            (int)a[16], (int)a[17], (int)a[18], op_ptr<float>(a[19]), (float)f[0], ctx->status)
  if (a[13] == GB_BF16) PREP(bf16); else PREP(float);
#undef PREP
  GB_CHECK_LAUNCH("latent_prep");
  return 1;
}

// a0 x (f32), a1 its row stride, a2 elements between heads in a row, a3 W [H, O, I], a4 its dtype, a5 out, a6 its
// dtype, a7 its row stride, a8 elements between heads in a row, a9 rows, a10 heads, a11 O, a12 I, a13 gate logits
// (f32, one per output element, laid out like a row of out) or 0: the outputs are multiplied by their sigmoid, a14
// their row stride; flags bit 0: the generic kernels whatever the sizes
GB_OP(gb_op_head_linear) {
  const int n = (int)a[9], H = (int)a[10], O = (int)a[11], I = (int)a[12];
  if (n <= 0) return 0;
  if (a[4] == GB_BF16 && !(flags & 1) &&
      gb_head_linear_tc_takes(n, I, a[1], a[2], op_ptr<const void>(a[0]), op_ptr<const void>(a[3]))) {
    gb_head_linear_tc_launch(op_ptr<const float>(a[0]), a[1], a[2], op_ptr<const bf16>(a[3]), op_ptr<void>(a[5]),
                             a[6] == GB_BF16, a[7], a[8], n, H, O, I, op_ptr<const float>(a[13]), a[14], ctx->stream);
    GB_CHECK_LAUNCH("head_linear (tensor cores)");
    return 1;
  }
  const bool small = n <= HL_SMALL_ROWS && (size_t)n * I * sizeof(float) <= 48 * 1024;
  const dim3 grid = small ? dim3(gb_div_up(O, 8), H) : dim3(gb_div_up(O, 64), gb_div_up(n, 64), H);
  const dim3 block(256);
  const size_t smem = small ? (size_t)n * I * sizeof(float) : 0;
#define HL(TW, TO)                                                                                                  \
  if (small)                                                                                                        \
    gb_launch(head_linear_small_kernel<TW, TO>, grid, block, smem, ctx->stream, op_ptr<const float>(a[0]), a[1], a[2], \
              op_ptr<const TW>(a[3]), op_ptr<TO>(a[5]), a[7], a[8], n, O, I, op_ptr<const float>(a[13]), a[14]);     \
  else                                                                                                              \
    gb_launch(head_linear_kernel<TW, TO>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], a[2],       \
              op_ptr<const TW>(a[3]), op_ptr<TO>(a[5]), a[7], a[8], n, O, I, op_ptr<const float>(a[13]), a[14])
  if (a[4] == GB_BF16) { if (a[6] == GB_BF16) { HL(bf16, bf16); } else { HL(bf16, float); } }
  else { if (a[6] == GB_BF16) { HL(float, bf16); } else { HL(float, float); } }
#undef HL
  GB_CHECK_LAUNCH("head_linear");
  return 1;
}

// a0 q' [tokens, heads, r + rot] (f32), a1 pages, a2 their dtype, a3 block table, a4 its entries per request, a5 page
// size, a6 number of pages, a7 token -> request, a8 token -> position, a9 gate logits (f32, [t, h] at a row stride) or
// 0, a10 that stride, a11 out [tokens, heads * r] (f32), a12 its row stride, a13 tokens, a14 heads, a15 latent size,
// a16 rotated size, a17 window (0: every earlier position), a18 longest context of the step (an upper bound will do),
// a19 workspace for partial results, gb_latent_attention_workspace_rows() rows of (latent size + 2) floats, a20 a
// learned sink score per head (f32 [heads]) whose exponential joins the softmax's denominator, or 0; a21 requests of
// the step, a22 first row per request (requests' rows follow one another in the order of the requests; a22 = 0: the
// generic kernel whatever the step); f0 scale
GB_OP(gb_op_latent_attention) {
  const int n = (int)a[13], H = (int)a[14], r = (int)a[15], dr = (int)a[16];
  if (n <= 0) return 0;
  // a step that carries portions of prompts, bfloat16 pages: the tensor-core kernel (latent_attention_tc.cu)
  if (a[22] &&
      gb_latent_attention_tc_takes(n, (int)a[21], H, r, dr, (int)a[17], a[2] == GB_BF16, op_ptr<const void>(a[1]),
                                   op_ptr<const void>(a[0]), op_ptr<const void>(a[11]), a[12])) {
    const int parts = gb_latent_attention_tc_launch(
        op_ptr<const float>(a[0]), op_ptr<const bf16>(a[1]), op_ptr<const int>(a[3]), (int)a[4], (int)a[5], (int)a[6],
        op_ptr<const int>(a[7]), op_ptr<const int>(a[8]), op_ptr<const int>(a[22]), op_ptr<const float>(a[9]), a[10],
        op_ptr<float>(a[11]), a[12], n, (int)a[21], H, r, dr, (float)f[0], op_ptr<const float>(a[20]), op_ptr<float>(a[19]),
        gb_latent_attention_workspace_rows(), ctx->status, ctx->stream);
    if (parts >= 1) {
      GB_CHECK_LAUNCH("latent_attention (tensor cores)");
      if (parts == 1) return 1;
      gb_launch(latent_attention_merge_kernel, dim3(gb_div_up((long long)n * H, 4)), dim3(128), 0, ctx->stream,
                op_ptr<const float>(a[19]), parts, op_ptr<const float>(a[9]), a[10], op_ptr<float>(a[11]), a[12], n, H, r,
                op_ptr<const float>(a[20]));
      GB_CHECK_LAUNCH("latent_attention_merge");
      return 2;
    }
  }
  if (r > 512) GB_FAIL(GB_ERR_ARG, "latent_attention: latent size %d (at most 512)", r);
  const int Dk = r + dr;
  if (dr > 32 * LA_RR) GB_FAIL(GB_ERR_ARG, "latent_attention: rotated size %d (at most %d)", dr, 32 * LA_RR);
  const size_t smem = sizeof(float) * (size_t)LA_KT * Dk;
  int chunk = 0;
  int splits = gb_latent_attention_chunks(n, H, (int)a[17], (int)a[18], &chunk);
  float* ws = op_ptr<float>(a[19]);
  if (ws == nullptr || (long long)n * H * splits > gb_latent_attention_workspace_rows()) splits = 1;
  // (fewer heads than a block has room for: fewer warps, so that none idles through the key tiles)
  const int warps = H >= LA_HB ? LA_WARPS : (gb_div_up(H, LA_HW) < 2 ? 2 : gb_div_up(H, LA_HW));
  const dim3 grid(n, gb_div_up(H, LA_HB), splits), block(32 * warps);
#define LA(TC, RL)                                                                                                   \
  do {                                                                                                               \
    static size_t allowed = 48 * 1024;     /* raised once per size, before any stream capture replays the launch */ \
    if (smem > allowed) {                                                                                            \
      GB_CUDA(cudaFuncSetAttribute(latent_attention_kernel<TC, RL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      allowed = smem;                                                                                                \
    }                                                                                                                \
    gb_launch(latent_attention_kernel<TC, RL>, grid, block, smem, ctx->stream, op_ptr<const float>(a[0]),             \
              op_ptr<const TC>(a[1]), op_ptr<const int>(a[3]), (int)a[4], (int)a[5], (int)a[6], op_ptr<const int>(a[7]), \
              op_ptr<const int>(a[8]), op_ptr<const float>(a[9]), a[10], op_ptr<float>(a[11]), a[12], H, r, dr,       \
              (float)f[0], (int)a[17], splits, chunk, ws, op_ptr<const float>(a[20]), ctx->status);                                              \
  } while (0)
#define LA_RL(TC)                                                                                                    \
  do {                                                                                                               \
    if (r <= 32) LA(TC, 1); else if (r <= 64) LA(TC, 2); else if (r <= 128) LA(TC, 4);                              \
    else if (r <= 256) LA(TC, 8); else LA(TC, 16);                                                                   \
  } while (0)
  if (a[2] == GB_BF16) LA_RL(bf16); else LA_RL(float);
#undef LA_RL
#undef LA
  GB_CHECK_LAUNCH("latent_attention");
  if (splits == 1) return 1;
  gb_launch(latent_attention_merge_kernel, dim3(gb_div_up((long long)n * H, 4)), dim3(128), 0, ctx->stream, ws, splits,
            op_ptr<const float>(a[9]), a[10], op_ptr<float>(a[11]), a[12], n, H, r, op_ptr<const float>(a[20]));
  GB_CHECK_LAUNCH("latent_attention_merge");
  return 2;
}
