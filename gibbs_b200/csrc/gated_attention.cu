// Grouped-query attention with keys and values of different widths, a norm over the WHOLE query (key)
// projection, a sliding window, a soft cap on the scores, a sink in the softmax and an output gate.
//
//  gb_op_embed_scaled    x[t, :] = table[id_t, :] * scale (32-bit)
//  gb_op_qk_prep         per token, from the 32-bit rows of the fused input product [q | k | v | ...]:
//                        q <- rot(rmsnorm_over_all_heads(q) * gain), the same for k, k and v written into the
//                        token's page; the norm is optional, the rotation turns the first `rot_dims` entries of
//                        every head in adjacent pairs (2i, 2i+1) by pos * inv_freq[i] (angle in 32-bit)
//  gb_op_sink_attention  out[t, h, :] = gate * sum_j p_j v_j over the visible keys j (0 <= pos - j < window, or
//                        all j <= pos), s_j = cap(scale * q . k_j), cap(s) = c * tanh(s / c) when c > 0,
//                        p_j = exp(s_j) / (sink + sum_i exp(s_i)) with sink = exp(z) when the softmax has a sink (a key
//                        of score z without a value: 0, or a learned number per head that is neither scaled nor
//                        capped) and 0 otherwise, gate = sigmoid(gate logit) per output element, or 1.  With
//                        `keep_first` > 0 a windowed position also sees the first `keep_first` positions of its
//                        sequence.  Scores, weights and sums are 32-bit.
//
// Pages: keys [n_pages, kv_heads, page_size, dim], values [n_pages, kv_heads, page_size, vdim].  A page id
// outside the pool is never dereferenced: the access is skipped and *status is set.
#include "hybrid.cuh"

namespace {

enum { STATUS_BAD_PAGE_WRITE = 1, STATUS_BAD_PAGE_READ = 2 };

// With a pair table: row (id before * mul_prev + id * mul_cur) mod buckets of it is added, row `buckets` for a
// sequence's first token.  The id before a portion's first token is the request's state (one int32 in its slot);
// the block of a portion's first row also leaves the portion's last id there, after it has read the old one.
template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int* ids, float* out, int dim, int vocab,
                                    float scale, const T* __restrict__ pairs, int buckets, long long mul_prev,
                                    long long mul_cur, const int* tok_req, const int* tok_pos, const int* q_start,
                                    const int* q_len, int* last, long long slot_stride, const int* slot_ids) {
  __shared__ int before;
  pdl_trigger();
  const int row = blockIdx.x;
  int r = 0, first = 0, pos = 0, count = 0;
  int* mine = nullptr;
  if (pairs) {
    r = tok_req[row];
    first = q_start[r];
    count = q_len[r];
    pos = tok_pos[row];
    mine = last + (size_t)slot_ids[r] * slot_stride;
  }
  pdl_wait();
  int id = __ldcg(ids + row);                       // (the kernel in front may have rewritten it)
  if (id < 0 || id >= vocab) id = 0;                // ids are checked on the host; a bad one reads row 0
  const T* src = table + (size_t)id * dim;
  float* dst = out + (size_t)row * dim;
  if (!pairs) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = to_f32(src[d]) * scale;
    return;
  }
  if (threadIdx.x == 0) {
    int b = -1;
    if (pos > 0) b = row > first ? __ldcg(ids + row - 1) : *mine;
    before = b;
    if (row == first) *mine = __ldcg(ids + first + count - 1);
  }
  __syncthreads();
  long long pr = buckets;
  if (before >= 0) pr = ((long long)before * mul_prev + (long long)id * mul_cur) % buckets;
  const T* add = pairs + (size_t)pr * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = fmaf(to_f32(src[d]), scale, to_f32(add[d]));
}

// How q and k are normed and turned (qk_prep's flags).
enum { PREP_NORM_WHOLE = 1, PREP_Q_BF16 = 2, PREP_PAGES_BF16 = 4, PREP_NORM_HEAD = 8, PREP_ROT_HALVES = 16,
       PREP_NORM_AFTER = 32 };

// One normed and rotated element of a projection: entry d of a head of `dim` entries that starts at `base`.
// `gain` is indexed like the projection (norm over the whole projection) or by d (`gain_per_head`: one gain
// vector shared by all heads).  The first `rot_dims` entries turn by pos * inv_freq[i], in adjacent pairs
// (2i, 2i+1) or, with `halves`, in pairs (i, i + rot_dims/2).
__device__ __forceinline__ float prep_element(const float* x, const float* __restrict__ gain, bool gain_per_head,
                                              float rstd, int base, int d, int rot_dims, bool halves,
                                              const float* __restrict__ inv_freq, int pos) {
  const int gb = gain_per_head ? 0 : base;
  const float own = x[base + d] * rstd * (gain ? gain[gb + d] : 1.f);
  if (d >= rot_dims) return own;
  const int half = rot_dims >> 1;
  const bool second = halves ? d >= half : (d & 1);
  const int partner = halves ? (second ? d - half : d + half) : (d ^ 1);
  const int fi = halves ? (second ? d - half : d) : (d >> 1);
  const float other = x[base + partner] * rstd * (gain ? gain[gb + partner] : 1.f);
  const float ang = (float)pos * inv_freq[fi];
  const float c = cosf(ang), s = sinf(ang);
  // the pair (u, v) becomes (u c - v s, v c + u s)
  return second ? own * c + other * s : own * c - other * s;
}

// One block per token.  A query head is `maps` heads of `dim` entries side by side (one for an ordinary
// attention), and so is a key head: a key row in the pages holds them all.  A warp takes one head of `dim`
// entries at a time: its norm (when heads are normed one by one), then its elements.
template <typename TC, typename TQ>
__global__ void qk_prep_kernel(const float* fused, long long ld, int k_col, int v_col, const float* __restrict__ q_gain,
                               const float* __restrict__ k_gain, const float* __restrict__ inv_freq, int rot_dims,
                               const int* tok_req, const int* tok_pos, const int* block_table, int bt_stride,
                               int page_size, TC* k_pages, TC* v_pages, int n_pages, int H, int G, int dim, int vdim,
                               int maps, int mode, float eps, TQ* q_out, long long ldq, int* status) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pos = tok_pos[t];
  const bool writes = k_pages != nullptr;
  const bool whole = mode & PREP_NORM_WHOLE, per_head = mode & PREP_NORM_HEAD, halves = mode & PREP_ROT_HALVES;
  // PREP_NORM_AFTER: every head is turned first and then divided by the root mean square of the TURNED head (no gain)
  const bool after = mode & PREP_NORM_AFTER;
  int page = -1;
  if (writes) page = block_table[(size_t)tok_req[t] * bt_stride + pos / page_size];
  pdl_wait();
  const float* row = fused + (size_t)t * ld;
  const int nq = H * maps * dim, nk = G * maps * dim;
  float q_rstd = 1.f, k_rstd = 1.f;
  if (whole) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) ss += row[i] * row[i];
    q_rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nq + eps);
    if (writes) {
      ss = 0.f;
      for (int i = threadIdx.x; i < nk; i += blockDim.x) ss += row[k_col + i] * row[k_col + i];
      k_rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)nk + eps);
    }
  }
  const bool normed = whole || per_head;
  for (int h = warp; h < H * maps; h += warps) {
    float rstd = q_rstd;
    if (per_head) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss += row[h * dim + d] * row[h * dim + d];
      rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
    }
    float post = 1.f;
    if (after) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) {
        const float v = prep_element(row, nullptr, true, 1.f, h * dim, d, rot_dims, halves, inv_freq, pos);
        ss += v * v;
      }
      post = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
    }
    for (int d = lane; d < dim; d += 32)
      q_out[(size_t)t * ldq + h * dim + d] = from_f32<TQ>(post * prep_element(row, normed ? q_gain : nullptr, per_head, rstd,
                                                                              h * dim, d, rot_dims, halves, inv_freq, pos));
  }
  if (!writes) return;
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) atomicExch(status, STATUS_BAD_PAGE_WRITE);
    return;
  }
  const int slot = pos % page_size;
  for (int h = warp; h < G * maps; h += warps) {
    const int g = h / maps, m = h - g * maps;
    float rstd = k_rstd;
    if (per_head) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss += row[k_col + h * dim + d] * row[k_col + h * dim + d];
      rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
    }
    TC* dst = k_pages + (((size_t)page * G + g) * page_size + slot) * ((size_t)maps * dim) + (size_t)m * dim;
    float post = 1.f;
    if (after) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) {
        const float v = prep_element(row + k_col, nullptr, true, 1.f, h * dim, d, rot_dims, halves, inv_freq, pos);
        ss += v * v;
      }
      post = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
    }
    for (int d = lane; d < dim; d += 32)
      dst[d] = from_f32<TC>(post * prep_element(row + k_col, normed ? k_gain : nullptr, per_head, rstd, h * dim, d, rot_dims,
                                                halves, inv_freq, pos));
  }
  for (int i = threadIdx.x; i < G * vdim; i += blockDim.x) {
    const int g = i / vdim, d = i - g * vdim;
    v_pages[(((size_t)page * G + g) * page_size + slot) * vdim + d] = from_f32<TC>(row[v_col + i]);
  }
}

// One block per (token, kv head and up to SA_WARPS of its query heads, chunk of keys); a warp looks after
// one query head.  Keys and values arrive in tiles of 32 positions in shared memory (32-bit), shared by the
// block's heads.  Lane j takes key j's score (the query is read from shared memory, the same address for
// all lanes; key rows lie an odd number of words apart); the tile's weights then enter the weighted sum of
// values with the lanes over the value's entries.  The sink joins at the end, by the same arithmetic as in
// the merge of chunks (sa_finish), so that a launch with one chunk and a launch with several whose other
// chunks are empty give the same bits.
constexpr int SA_WARPS = 8, SA_KT = 32;

// The sums over chunks s of exp(m_s - M) * (l_s, acc_s) with M = max(m_s, the sink's score): what both the
// attention kernel (one chunk) and the merge kernel (several) divide by and multiply with.
// (z: the sink's score, 0 unless the heads have learned ones)
__device__ __forceinline__ float sa_sink_score(const float* __restrict__ scores, int head) { return scores ? scores[head] : 0.f; }
__device__ __forceinline__ float sa_top(float m, int sink, float z) { return sink ? fmaxf(m, z) : m; }
__device__ __forceinline__ float sa_sink_weight(float M, int sink, float z) { return sink ? expf(z - M) : 0.f; }

template <typename TC, typename TQ, typename TO, int VR>
__global__ void __launch_bounds__(32 * SA_WARPS)
sink_attention_kernel(const TQ* q, long long ldq, const TC* k_pages, const TC* v_pages, const int* block_table,
                      int bt_stride, int page_size, int n_pages, const int* tok_req, const int* tok_pos,
                      const float* gate, long long ld_gate, TO* out, long long ldo, int H, int G, int dim, int vdim,
                      float scale, float softcap, int window, int sink, int splits, int chunk, float* ws, int maps,
                      int blocked, const float* __restrict__ sink_scores, int keep_first, int* status) {
  // (H counts heads of `dim` entries: `maps` of them make one query head, and a key row holds `maps` keys side
  // by side, of which head h scores against number h % maps)
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  const int group = H / G;
  const int hb = (group + SA_WARPS - 1) / SA_WARPS;          // blocks per kv head
  const int g = blockIdx.y / hb, h_first = g * group + (blockIdx.y - g * hb) * SA_WARPS;
  const int warps = blockDim.x >> 5;
  const int KD = maps * dim;                                  // entries of a key row
  const int KS = KD | 1;                                      // words between key rows: odd
  long long* src = reinterpret_cast<long long*>(sm);          // [SA_KT] row of each key of the tile in the pages
  float* qs = sm + 2 * SA_KT;                                 // [warps][dim]
  float* ks = qs + warps * dim;                               // [SA_KT][KS]
  float* vs = ks + SA_KT * KS;                                // [SA_KT][vdim]
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = h_first + warp;
  const bool live = h < (g + 1) * group;
  const int pos = tok_pos[t];
  const int* table = block_table + (size_t)tok_req[t] * bt_stride;
  // visible: the last `window` positions, or (`blocked`) the positions of pos's own block of `window`
  const int lo = window > 0 ? (blocked ? (pos / window) * window : max(0, pos - window + 1)) : 0;
  // the visible keys in order: the first `kept` positions of the sequence that lie in front of the window, then
  // lo .. pos; key number v of this list is position v (v < kept) or lo + v - kept
  const int kept = window > 0 ? min(keep_first, lo) : 0;
  const int shift = lo - kept;
  const int k_last = kept + pos - lo;
  const int k_begin = splits > 1 ? (int)blockIdx.z * chunk : 0;
  const int k_end = splits > 1 ? min(k_last, k_begin + chunk - 1) : k_last;
  pdl_wait();
  for (int i = threadIdx.x; i < warps * dim; i += blockDim.x) {
    const int w = i / dim, d = i - w * dim;
    const int hh = h_first + w;
    qs[i] = hh < (g + 1) * group ? to_f32(q[(size_t)t * ldq + (size_t)hh * dim + d]) : 0.f;
  }
  float acc[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int k0 = k_begin; k0 <= k_end; k0 += SA_KT) {
    __syncthreads();                                          // the last tile has been used (and qs is written)
    if (threadIdx.x < SA_KT) {
      const int kv = k0 + threadIdx.x;
      const int kp = kv < kept ? kv : kv + shift;
      long long at = -1;
      if (kv <= k_end) {
        const int page = table[kp / page_size];
        if (page < 0 || page >= n_pages) atomicExch(status, STATUS_BAD_PAGE_READ);
        else at = ((long long)page * G + g) * page_size + kp % page_size;
      }
      src[threadIdx.x] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < SA_KT * KD; i += blockDim.x) {
      const int j = i / KD, d = i - j * KD;
      ks[j * KS + d] = src[j] >= 0 ? to_f32(k_pages[(size_t)src[j] * KD + d]) : 0.f;
    }
    for (int i = threadIdx.x; i < SA_KT * vdim; i += blockDim.x) {
      const int j = i / vdim, d = i - j * vdim;
      vs[i] = src[j] >= 0 ? to_f32(v_pages[(size_t)src[j] * vdim + d]) : 0.f;
    }
    __syncthreads();
    if (!live) continue;
    const float* qh = qs + warp * dim;
    const float* kr = ks + lane * KS + (h % maps) * dim;
    float s0 = 0.f, s1 = 0.f;                                 // two chains, added in a fixed order
    int d = 0;
    for (; d + 1 < dim; d += 2) {
      s0 = fmaf(qh[d], kr[d], s0);
      s1 = fmaf(qh[d + 1], kr[d + 1], s1);
    }
    if (d < dim) s0 = fmaf(qh[d], kr[d], s0);
    float s = (s0 + s1) * scale;
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    if (k0 + lane > k_end) s = -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;                         // (cannot happen: a tile holds a visible key)
    const float corr = expf(m - m_new);                 // 0 while m = -inf
    const float p = expf(s - m_new);                    // 0 for a key that is not seen
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[i] *= corr;
    const int n_keys = min(SA_KT, k_end - k0 + 1);
    for (int j = 0; j < n_keys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const int dv = lane + 32 * i;
        if (dv < vdim) acc[i] = fmaf(pj, vs[j * vdim + dv], acc[i]);
      }
    }
  }
  if (!live) return;
  if (splits > 1) {
    float* w = ws + (((size_t)t * H + h) * splits + blockIdx.z) * (vdim + 2);
    if (lane == 0) { w[0] = m; w[1] = l; }
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int dv = lane + 32 * i;
      if (dv < vdim) w[2 + dv] = acc[i];
    }
    return;
  }
  const float z = sa_sink_score(sink_scores, h / maps);
  const float M = sa_top(m, sink, z);
  const float e = expf(m - M);
  const float inv = 1.0f / fmaf(e, l, sa_sink_weight(M, sink, z));
#pragma unroll
  for (int i = 0; i < VR; ++i) {
    const int dv = lane + 32 * i;
    if (dv < vdim) {
      const float gt = gate ? hy_sigmoid(gate[(size_t)t * ld_gate + (size_t)h * vdim + dv]) : 1.f;
      out[(size_t)t * ldo + (size_t)h * vdim + dv] = from_f32<TO>(fmaf(e, acc[i], 0.f) * inv * gt);
    }
  }
}

// One warp per (token, head): the chunks' partial results (maximum, sum of weights, weighted sum), merged in
// chunk order; the sink joins as a chunk of maximum 0, weight 1 and no values.
template <typename TO>
__global__ void sink_attention_merge_kernel(const float* ws, int splits, const float* gate, long long ld_gate, TO* out,
                                            long long ldo, int n, int H, int vdim, int sink,
                                            const float* __restrict__ sink_scores, int maps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= (long long)n * H) return;
  const int t = (int)(idx / H), h = (int)(idx - (long long)t * H);
  const float* w = ws + (size_t)idx * splits * (vdim + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, w[(size_t)s * (vdim + 2)]);
  const float z = sa_sink_score(sink_scores, h / maps);
  M = sa_top(M, sink, z);
  float L = sa_sink_weight(M, sink, z);
  for (int s = 0; s < splits; ++s) {
    const float ms = w[(size_t)s * (vdim + 2)];
    if (ms > -INFINITY) L = fmaf(expf(ms - M), w[(size_t)s * (vdim + 2) + 1], L);
  }
  const float inv = 1.0f / L;
  for (int dv = lane; dv < vdim; dv += 32) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = w[(size_t)s * (vdim + 2)];
      if (ms > -INFINITY) a = fmaf(expf(ms - M), w[(size_t)s * (vdim + 2) + 2 + dv], a);
    }
    const float gt = gate ? hy_sigmoid(gate[(size_t)t * ld_gate + (size_t)h * vdim + dv]) : 1.f;
    out[(size_t)t * ldo + (size_t)h * vdim + dv] = from_f32<TO>(a * inv * gt);
  }
}

constexpr int SA_WS_ROWS = 1 << 16;

}  // namespace

// Rows of (vdim + 2) floats a launch's partial results may need, whatever its sizes.
GB_API int gb_sink_attention_workspace_rows() { return SA_WS_ROWS; }

// The merge of chunks, for this file's kernel and for the tensor-core one (gated_attention_tc.cu).
int gb_sink_attention_merge(const float* ws, int splits, const float* gate, long long ld_gate, void* out, int out_bf16,
                            long long ldo, int n, int H, int vdim, int sink, const float* sink_scores, int maps,
                            cudaStream_t stream) {
  const dim3 mgrid(gb_div_up((long long)n * H, 4));
  if (out_bf16)
    gb_launch(sink_attention_merge_kernel<bf16>, mgrid, dim3(128), 0, stream, ws, splits, gate, ld_gate, (bf16*)out, ldo, n,
              H, vdim, sink, sink_scores, maps);
  else
    gb_launch(sink_attention_merge_kernel<float>, mgrid, dim3(128), 0, stream, ws, splits, gate, ld_gate, (float*)out, ldo,
              n, H, vdim, sink, sink_scores, maps);
  GB_CHECK_LAUNCH("sink_attention_merge");
  return 1;
}

// How the visible keys of a launch are cut into chunks of whole key tiles: (chunks, keys per chunk).  Few
// tokens (decoding) get many chunks, so that the GPU is occupied.  Chunks lie at fixed distances from the
// first visible key, so a chunk's partial result does not depend on how many chunks there are.
GB_API int gb_sink_attention_chunks(int n, int H, int G, int window, int max_ctx, int* chunk_out) {
  // (`window`: the most keys a windowed position sees, the kept first positions included)
  const int group = H / (G > 0 ? G : 1);
  const int blocks = n * G * gb_div_up(group, SA_WARPS);
  int wanted = 592 / (blocks > 0 ? blocks : 1);
  if (wanted > 64) wanted = 64;
  const int span = window > 0 ? window : (max_ctx > 0 ? max_ctx : 1);
  // (with a window the cut depends on the launch's sizes only, not on how long the contexts are)
  if (wanted <= 1 || (window > 0 && span <= SA_KT)) { *chunk_out = span; return 1; }
  int chunk;
  if (window > 0) {
    chunk = SA_KT * gb_div_up(gb_div_up(span, wanted), SA_KT);
  } else {
    chunk = 256;
    while (gb_div_up(span, chunk) > 2 * wanted) chunk *= 2;
  }
  *chunk_out = chunk;
  return gb_div_up(span, chunk);
}

// a0 table, a1 its dtype, a2 token ids, a3 out (f32 [tokens, dim]), a4 tokens, a5 dim, a6 vocabulary; with a pair
// table: a7 the table [buckets + 1, dim] (same dtype) or 0, a8 buckets, a9 factor of the id before, a10 factor of the
// id, a11 token -> request, a12 token -> position, a13 first row per request, a14 rows per request, a15 the id
// before (int32, one per slot) of slot 0, a16 elements between slots, a17 slot ids; f0 scale
GB_OP(gb_op_embed_scaled) {
  const int n = (int)a[4], dim = (int)a[5];
  if (n <= 0) return 0;
  if (a[7] && a[8] <= 0) GB_FAIL(GB_ERR_ARG, "embed_scaled: a pair table of %lld buckets", a[8]);
  const dim3 block(dim >= 1024 ? 256 : 128);
#define EMBED(T)                                                                                                        \
  gb_launch(embed_scaled_kernel<T>, dim3(n), block, 0, ctx->stream, op_ptr<const T>(a[0]), op_ptr<const int>(a[2]),      \
            op_ptr<float>(a[3]), dim, (int)a[6], (float)f[0], op_ptr<const T>(a[7]), (int)a[8], a[9], a[10],              \
            op_ptr<const int>(a[11]), op_ptr<const int>(a[12]), op_ptr<const int>(a[13]), op_ptr<const int>(a[14]),      \
            op_ptr<int>(a[15]), a[16], op_ptr<const int>(a[17]))
  if (a[1] == GB_BF16) EMBED(bf16); else EMBED(float);
#undef EMBED
  GB_CHECK_LAUNCH("embed_scaled");
  return 1;
}

// a0 fused rows (f32) [q (heads * maps * dim) | ...], a1 their stride, a2 column of the keys (kv_heads * maps * dim),
// a3 column of the values (kv_heads * vdim), a4 gain of the query norm or 0, a5 gain of the key norm or 0, a6 inv_freq
// [rot_dims / 2], a7 rot_dims, a8 token -> request, a9 token -> position, a10 block table, a11 its entries per request,
// a12 page size, a13 key pages or 0 (a layer that reads another layer's cache writes none), a14 value pages, a15 number
// of pages, a16 tokens, a17 heads, a18 kv heads, a19 dim, a20 vdim, a21 q out [tokens, heads * maps * dim], a22 maps
// (heads of `dim` entries side by side in one query or key head; 0 means 1); flags bit 0: norm over the whole
// projection (gains as long as the projection), bit 1: q out is bfloat16 (else 32-bit), bit 2: the pages are bfloat16,
// bit 3: norm over every head of `dim` entries (gains of `dim` entries, shared), bit 4: the rotation pairs entry i
// with entry i + rot_dims / 2 (else adjacent entries), bit 5: every head of `dim` entries is divided by its root mean
// square AFTER the rotation, without a gain; f0 eps
GB_OP(gb_op_qk_prep) {
  const int n = (int)a[16], H = (int)a[17], G = (int)a[18], dim = (int)a[19], vdim = (int)a[20];
  const int maps = a[22] > 0 ? (int)a[22] : 1;
  if (n <= 0) return 0;
  if (a[7] % 2 || a[7] > dim) GB_FAIL(GB_ERR_ARG, "qk_prep: %lld rotated dimensions of %d", a[7], dim);
  if (G <= 0 || H % G) GB_FAIL(GB_ERR_ARG, "qk_prep: %d heads over %d kv heads", H, G);
  if (((flags & PREP_NORM_WHOLE) ? 1 : 0) + ((flags & PREP_NORM_HEAD) ? 1 : 0) + ((flags & PREP_NORM_AFTER) ? 1 : 0) > 1)
    GB_FAIL(GB_ERR_ARG, "qk_prep: one kind of norm at a time");
  const int threads = H * maps * dim >= 2048 ? 512 : 256;
  const long long ldq = (long long)H * maps * dim;
  const int mode = flags & (PREP_NORM_WHOLE | PREP_NORM_HEAD | PREP_ROT_HALVES | PREP_NORM_AFTER);
#define PREP(TC, TQ)                                                                                                     \
  gb_launch(qk_prep_kernel<TC, TQ>, dim3(n), dim3(threads), 0, ctx->stream, op_ptr<const float>(a[0]), a[1], (int)a[2],    \
            (int)a[3], op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), op_ptr<const float>(a[6]), (int)a[7],        \
            op_ptr<const int>(a[8]), op_ptr<const int>(a[9]), op_ptr<const int>(a[10]), (int)a[11], (int)a[12],           \
            op_ptr<TC>(a[13]), op_ptr<TC>(a[14]), (int)a[15], H, G, dim, vdim, maps, mode, (float)f[0], op_ptr<TQ>(a[21]), \
            ldq, ctx->status)
  if (flags & PREP_PAGES_BF16) { if (flags & PREP_Q_BF16) PREP(bf16, bf16); else PREP(bf16, float); }
  else { if (flags & PREP_Q_BF16) GB_FAIL(GB_ERR_ARG, "qk_prep: bfloat16 queries with 32-bit pages"); PREP(float, float); }
#undef PREP
  GB_CHECK_LAUNCH("qk_prep");
  return 1;
}

// a0 q [tokens, heads * maps * dim], a1 key pages, a2 value pages, a3 block table, a4 its entries per request, a5 page
// size, a6 number of pages, a7 token -> request, a8 token -> position, a9 gate logits (f32, [t, heads * vdim] at a row
// stride) or 0, a10 that stride, a11 out [tokens, heads * maps * vdim], a12 its row stride, a13 tokens, a14 heads, a15 kv
// heads, a16 dim, a17 vdim, a18 window (0: every earlier position), a19 longest context of the step (an upper bound
// will do), a20 workspace for partial results (gb_sink_attention_workspace_rows() rows of vdim + 2 floats) or 0, a21
// maps (0 means 1): a query head is `maps` heads of `dim` entries, a key row [maps * dim] holds one key for each, all
// share the value; every map is a softmax of its own and has an output of its own;
// flags bit 0: the softmax has a sink, bit 1: q is bfloat16 (else 32-bit), bit 2: the pages are, bit 3: out is,
// bit 4: position p sees the positions of its own block of `window` positions, counted from 0, up to p (else
// the last `window`); a22 a learned score of the sink per head (f32 [heads]) or 0: the sink's score is 0;
// f0 scale, f1 soft cap (0: none), f2 keep_first: a windowed position also sees the positions below this number
GB_OP(gb_op_sink_attention) {
  const int n = (int)a[13], G = (int)a[15], dim = (int)a[16], vdim = (int)a[17];
  const int maps = a[21] > 0 ? (int)a[21] : 1;
  const int H = (int)a[14] * maps;
  if (n <= 0) return 0;
  if (G <= 0 || a[14] % G) GB_FAIL(GB_ERR_ARG, "sink_attention: %lld heads over %d kv heads", a[14], G);
  if (vdim > 256) GB_FAIL(GB_ERR_ARG, "sink_attention: values of %d entries (at most 256)", vdim);
  const int group = H / G, sink = flags & 1, blocked = (flags & 16) ? 1 : 0;
  if (blocked && a[18] <= 0) GB_FAIL(GB_ERR_ARG, "sink_attention: blocks of %lld positions", a[18]);
  const int keep_first = a[18] > 0 ? (int)f[2] : 0;
  if (keep_first < 0 || (keep_first > 0 && blocked)) GB_FAIL(GB_ERR_ARG, "sink_attention: %d kept first positions", keep_first);
  if (a[22] && !sink) GB_FAIL(GB_ERR_ARG, "sink_attention: learned sink scores without a sink");
  const float* sink_scores = op_ptr<const float>(a[22]);
  const int warps = group < SA_WARPS ? group : SA_WARPS;
  const int hb = gb_div_up(group, SA_WARPS);
  const int KS = (maps * dim) | 1;
  const size_t smem = sizeof(long long) * SA_KT + sizeof(float) * ((size_t)warps * dim + (size_t)SA_KT * (KS + vdim));
  if (smem > 200 * 1024) GB_FAIL(GB_ERR_ARG, "sink_attention: heads of %d entries need %zu bytes of shared memory", dim, smem);
  int chunk = 0;
  int splits = gb_sink_attention_chunks(n, H, G, a[18] > 0 ? (int)a[18] + keep_first : 0, (int)a[19], &chunk);
  float* ws = op_ptr<float>(a[20]);
  if (ws == nullptr || (long long)n * H * splits > SA_WS_ROWS) splits = 1;
  const dim3 grid(n, G * hb, splits), block(32 * warps);
#define SA(TC, TQ, TO, VR)                                                                                              \
  do {                                                                                                                  \
    static size_t allowed = 48 * 1024;     /* raised once per size, before any stream capture replays the launch */    \
    if (smem > allowed) {                                                                                               \
      GB_CUDA(cudaFuncSetAttribute(sink_attention_kernel<TC, TQ, TO, VR>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                   (int)smem));                                                                         \
      allowed = smem;                                                                                                   \
    }                                                                                                                   \
    gb_launch(sink_attention_kernel<TC, TQ, TO, VR>, grid, block, smem, ctx->stream, op_ptr<const TQ>(a[0]),             \
              (long long)H * dim, op_ptr<const TC>(a[1]), op_ptr<const TC>(a[2]), op_ptr<const int>(a[3]), (int)a[4],    \
              (int)a[5], (int)a[6], op_ptr<const int>(a[7]), op_ptr<const int>(a[8]), op_ptr<const float>(a[9]), a[10],  \
              op_ptr<TO>(a[11]), a[12], H, G, dim, vdim, (float)f[0], (float)f[1], (int)a[18], sink, splits, chunk, ws,  \
              maps, blocked, sink_scores, keep_first, ctx->status);                                                    \
  } while (0)
#define SA_VR(TC, TQ, TO)                                                                                               \
  do {                                                                                                                  \
    if (vdim <= 32) SA(TC, TQ, TO, 1); else if (vdim <= 64) SA(TC, TQ, TO, 2); else if (vdim <= 128) SA(TC, TQ, TO, 4); \
    else SA(TC, TQ, TO, 8);                                                                                             \
  } while (0)
  const bool qb = flags & 2, cb = flags & 4, ob = flags & 8;
  if (cb && qb && ob) SA_VR(bf16, bf16, bf16);
  else if (cb && !qb && ob) SA_VR(bf16, float, bf16);
  else if (cb && !qb && !ob) SA_VR(bf16, float, float);
  else if (!cb && !qb && !ob) SA_VR(float, float, float);
  else GB_FAIL(GB_ERR_ARG, "sink_attention: this combination of query, page and output types is not built");
#undef SA_VR
#undef SA
  GB_CHECK_LAUNCH("sink_attention");
  if (splits == 1) return 1;
  const int rc = gb_sink_attention_merge(ws, splits, op_ptr<const float>(a[9]), a[10], op_ptr<void>(a[11]), ob ? 1 : 0, a[12],
                                         n, H, vdim, sink, sink_scores, maps, ctx->stream);
  return rc < 0 ? rc : 2;
}
