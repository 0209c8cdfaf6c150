// A feed-forward that routes every token to `top` of E experts.
//
//  gb_op_moe_route     per token: the `top` largest router logits (ties: the lower index), their
//                      sigmoids as weights (not renormalised), and the sigmoid of the shared expert's
//                      gate logit; all in 32-bit
//  gb_op_moe_route_grouped  the same choice for routers with softmax (or sigmoid) scores, a correction added to
//                      the scores for the choice only, experts in groups of which only the best are open, and
//                      trailing "identity" outputs that stand for experts returning their input
//  gb_op_moe_sort      (token, choice) pairs ordered by expert: offsets[E + 1], the pair behind every
//                      row, the row of every pair
//  gb_op_moe_gather    rows[row] = weight * h[token]: the weight multiplies the expert's INPUT
//  gb_op_moe_experts   per expert, over its rows: either act = glu(rows W_gate^T, rows W_up^T) with
//                      clamps, or out = rows W_down^T (32-bit)
//  gb_op_moe_combine   y[token] = sum over its choices of out[row] (+ gate * shared[token])
//  gb_op_moe_combine_weighted  y[token] (+)= sum over its choices of weight * out[row], where the weight multiplies
//                      the expert's OUTPUT; a choice beyond the real experts contributes weight * h[token]
//
// A row's result does not depend on which rows share its tile (one accumulator per output walking k
// upwards), so the order in which pairs land inside an expert's range does not matter.
#include "hybrid.cuh"

namespace {

constexpr int MOE_MAX_EXPERTS = 1024;

// one warp per token: lane l looks after experts l, l + 32, ... (a bit per expert it has given away)
__global__ void moe_route_kernel(const float* logits, long long ld, int n, int E, int top, int shared_col, int* idx,
                                 float* weight, float* shared_gate) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n) return;
  const float* z = logits + (size_t)t * ld;
  unsigned taken = 0;
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int i = 0, e = lane; e < E; ++i, e += 32) {
      if ((taken >> i) & 1u) continue;
      const float v = z[e];
      if (v > bv || be == 0x7fffffff) { bv = v; be = e; }   // (ascending e: a tie keeps the lower index)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    if ((be & 31) == lane) taken |= 1u << (be >> 5);
    if (lane == 0) {
      idx[(size_t)t * top + k] = be;
      weight[(size_t)t * top + k] = hy_sigmoid(bv);
    }
  }
  if (shared_gate && lane == 0) shared_gate[t] = hy_sigmoid(z[shared_col]);
}

// One warp per token.  scores: 0 sigmoid(z), 1 softmax(z) over all `n_out` router outputs, 2 the logits z themselves.
// `normalise`: 0 a chosen output's weight is its score, 1 the score divided by the sum of the chosen scores, 2 the
// softmax over the chosen scores alone.  The choice is made on
// score + correction; with `groups` > 1 the outputs form that many equal groups of neighbours, a group's mark is
// its largest choice score, and only outputs of the `keep` best groups can be chosen.  The weight of a chosen
// output is its score without the correction, not renormalised.  Ties go to the lower index.
__global__ void moe_route_grouped_kernel(const float* logits, long long ld, int n, int n_out, int top, int scores,
                                         const float* __restrict__ correction, int groups, int keep, int* idx,
                                         float* weight, int normalise) {
  extern __shared__ float route_sm[];                    // per warp: scores [n_out], choice scores [n_out], group marks
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  float* s = route_sm + (size_t)warp * (2 * n_out + groups);
  float* c = s + n_out;
  float* mark = c + n_out;
  const float* z = logits + (size_t)t * ld;
  if (scores == 1) {
    float mx = -INFINITY;
    for (int e = lane; e < n_out; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_out; e += 32) {
      const float v = expf(z[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < n_out; e += 32) s[e] = s[e] / sum;
  } else if (scores == 2) {
    for (int e = lane; e < n_out; e += 32) s[e] = z[e];
  } else {
    for (int e = lane; e < n_out; e += 32) s[e] = hy_sigmoid(z[e]);
  }
  for (int e = lane; e < n_out; e += 32) c[e] = s[e] + (correction ? correction[e] : 0.f);
  __syncwarp();
  const int gs = n_out / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float b = -INFINITY;
      for (int e = g * gs; e < (g + 1) * gs; ++e) b = fmaxf(b, c[e]);
      mark[g] = b;
    }
    __syncwarp();
    // the `keep` best groups stay open: the mark of a group that is picked becomes +infinity, which no score
    // reaches, so that the pass below reads one flag per group
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY;
      int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = mark[g];
        if (v != INFINITY && (bg == 0x7fffffff || v > bv)) { bv = v; bg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (og != 0x7fffffff && (bg == 0x7fffffff || ov > bv || (ov == bv && og < bg))) { bv = ov; bg = og; }
      }
      if (lane == 0 && bg != 0x7fffffff) mark[bg] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_out; e += 32)
      if (mark[e / gs] != INFINITY) c[e] = -INFINITY;     // (a closed output; an open one keeps its own score)
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < n_out; e += 32) {
      const float v = c[e];
      if (v != -INFINITY || be == 0x7fffffff)
        if (be == 0x7fffffff || v > bv) { bv = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    if (lane == 0) {
      idx[(size_t)t * top + k] = be;
      weight[(size_t)t * top + k] = s[be];
      c[be] = -INFINITY;                                   // taken
    }
    __syncwarp();
  }
  if (normalise && lane == 0) {
    float* w = weight + (size_t)t * top;
    float sum = 0.f;
    if (normalise == 2) {
      const float mx = w[0];                                // (the first choice has the largest score)
      for (int k = 0; k < top; ++k) {
        w[k] = expf(w[k] - mx);
        sum += w[k];
      }
    } else {
      for (int k = 0; k < top; ++k) sum += w[k];
    }
    for (int k = 0; k < top; ++k) w[k] = w[k] / sum;
  }
}

// one block
__global__ void moe_sort_kernel(const int* idx, int pairs, int E, int* offsets, int* row_pair, int* pair_row) {
  __shared__ int count[MOE_MAX_EXPERTS + 1];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      const int c = count[e];
      offsets[e] = at;
      count[e] = at;
      at += c;
    }
    offsets[E] = at;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int row = atomicAdd(&count[idx[p]], 1);
    row_pair[row] = p;
    pair_row[p] = row;
  }
}

template <typename T>
__global__ void moe_gather_kernel(const T* h, long long ldh, const int* row_pair, const float* weight, T* rows,
                                  long long ldr, int pairs, int width, int top) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int p = row_pair[row];
  const float w = weight ? weight[p] : 1.f;              // (no weights: they multiply the experts' outputs instead)
  const T* src = h + (size_t)(p / top) * ldh;
  T* dst = rows + (size_t)row * ldr;
  for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = from_f32<T>(w * to_f32(src[d]));
}

// The block's (expert, first row) among the tiles of all experts' ranges, or false.
__device__ __forceinline__ bool moe_tile(const int* offsets, int E, int tile, int& e, int& r0, int& r1) {
  for (e = 0; e < E; ++e) {
    const int lo = offsets[e], hi = offsets[e + 1];
    const int tiles = (hi - lo + 63) >> 6;
    if (tile < tiles) {
      r0 = lo + 64 * tile;
      r1 = hi;
      return true;
    }
    tile -= tiles;
  }
  return false;
}

// GLU: tile columns alternate gate, up, gate, up, ... of 32 features; out [rows, ff]
template <typename TA, typename TW>
__global__ void moe_experts_glu_kernel(const TA* rows, long long ldr, const TW* __restrict__ W, const int* offsets, int E,
                                       TA* act, long long lda, int ff, int width, float alpha, float limit, float up_add,
                                       int blocks64) {
  pdl_trigger();
  pdl_wait();
  int e, r0, r1;
  if (!moe_tile(offsets, E, blockIdx.y, e, r0, r1)) return;
  const int c0 = blockIdx.x * 32;
  const TW* wb = W + (size_t)e * 2 * ff * width;       // [gate rows (ff) | up rows (ff)]
  float acc[4][4];
  int ty, tx;
  hy_tile_64x64<TA, TW>(
      [&](int i) -> const TA* { return r0 + i < r1 ? rows + (size_t)(r0 + i) * ldr : nullptr; },
      [&](int j) -> const TW* {
        const int c = c0 + (j >> 1);
        // rows [gate (ff) | up (ff)], or alternating in blocks of 64: gate 0-63, up 0-63, gate 64-127, ...
        const size_t wrow = blocks64 ? (size_t)(c >> 6) * 128 + (j & 1) * 64 + (c & 63) : (size_t)(j & 1) * ff + c;
        return c < ff ? wb + wrow * width : nullptr;
      },
      width, acc, ty, tx);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = r0 + ty * 4 + r;
    if (row >= r1) continue;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int col = c0 + tx * 2 + c;
      if (col < ff)
        act[(size_t)row * lda + col] = from_f32<TA>(hy_clamped_glu(acc[r][2 * c], acc[r][2 * c + 1], alpha, limit, up_add));
    }
  }
}

template <typename TA, typename TW>
__global__ void moe_experts_down_kernel(const TA* act, long long lda, const TW* __restrict__ W, const int* offsets, int E,
                                        float* out, long long ldo, int width, int ff) {
  pdl_trigger();
  pdl_wait();
  int e, r0, r1;
  if (!moe_tile(offsets, E, blockIdx.y, e, r0, r1)) return;
  const int c0 = blockIdx.x * 64;
  const TW* wb = W + (size_t)e * width * ff;
  float acc[4][4];
  int ty, tx;
  hy_tile_64x64<TA, TW>(
      [&](int i) -> const TA* { return r0 + i < r1 ? act + (size_t)(r0 + i) * lda : nullptr; },
      [&](int j) -> const TW* { return c0 + j < width ? wb + (size_t)(c0 + j) * ff : nullptr; }, ff, acc, ty, tx);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = r0 + ty * 4 + r;
    if (row >= r1) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = c0 + tx * 4 + c;
      if (col < width) out[(size_t)row * ldo + col] = acc[r][c];
    }
  }
}

__global__ void moe_combine_kernel(const float* out, long long ldo, const int* pair_row, const float* shared_gate,
                                   const float* shared, long long lds, float* y, long long ldy, int width, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float g = shared_gate ? shared_gate[t] : 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) v += out[(size_t)pair_row[(size_t)t * top + k] * ldo + d];
    if (shared) v += g * shared[(size_t)t * lds + d];
    y[(size_t)t * ldy + d] = v;
  }
}

template <typename T>
__global__ void moe_combine_weighted_kernel(const float* out, long long ldo, const int* pair_row, const int* idx,
                                            const float* weight, const T* h, long long ldh, float* y, long long ldy,
                                            int width, int top, int E, int accumulate) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t p = (size_t)t * top + k;
      const float src = idx[p] < E ? out[(size_t)pair_row[p] * ldo + d] : to_f32(h[(size_t)t * ldh + d]);
      v = fmaf(weight[p], src, v);
    }
    float* o = y + (size_t)t * ldy + d;
    *o = accumulate ? *o + v : v;
  }
}

}  // namespace

// a0 logits (f32), a1 their row stride, a2 tokens, a3 router outputs (experts and identity outputs), a4 top, a5 scores
// (0 sigmoid, 1 softmax, 2 the logits), a6 correction [outputs] (f32) or 0, a7 groups (1: none), a8 groups kept, a9 chosen
// outputs [tokens, top] (int32), a10 their weights (f32), a11 how the chosen scores become weights: 0 as they are, 1
// divided by their sum, 2 their softmax
GB_OP(gb_op_moe_route_grouped) {
  const int n = (int)a[2], n_out = (int)a[3], top = (int)a[4];
  int groups = (int)a[7], keep = (int)a[8];
  if (n <= 0) return 0;
  if (groups < 1) groups = 1;
  if (keep < 1 || keep > groups) keep = groups;
  if (n_out > MOE_MAX_EXPERTS) GB_FAIL(GB_ERR_ARG, "moe_route_grouped: %d router outputs (at most %d)", n_out, MOE_MAX_EXPERTS);
  if (n_out % groups) GB_FAIL(GB_ERR_ARG, "moe_route_grouped: %d router outputs in %d groups", n_out, groups);
  if (top < 1 || top > (n_out / groups) * keep)
    GB_FAIL(GB_ERR_ARG, "moe_route_grouped: top %d of the %d outputs in %d open groups", top, (n_out / groups) * keep, keep);
  const int warps = 4;
  const size_t smem = sizeof(float) * warps * (2 * (size_t)n_out + groups);
  gb_launch(moe_route_grouped_kernel, dim3(gb_div_up(n, warps)), dim3(32 * warps), smem, ctx->stream,
            op_ptr<const float>(a[0]), a[1], n, n_out, top, (int)a[5], op_ptr<const float>(a[6]), groups, keep,
            op_ptr<int>(a[9]), op_ptr<float>(a[10]), (int)a[11]);
  GB_CHECK_LAUNCH("moe_route_grouped");
  return 1;
}

// a0 logits (f32), a1 their row stride, a2 tokens, a3 experts, a4 top, a5 column of the shared expert's gate logit,
// a6 chosen experts [tokens, top] (int32), a7 their weights (f32), a8 shared gate [tokens] (f32), or 0 for none
GB_OP(gb_op_moe_route) {
  const int n = (int)a[2], E = (int)a[3], top = (int)a[4];
  if (n <= 0) return 0;
  if (top < 1 || top > E) GB_FAIL(GB_ERR_ARG, "moe_route: top %d of %d experts", top, E);
  if (E > MOE_MAX_EXPERTS) GB_FAIL(GB_ERR_ARG, "moe_route: %d experts (at most %d)", E, MOE_MAX_EXPERTS);
  gb_launch(moe_route_kernel, dim3(gb_div_up(n, 4)), dim3(128), 0, ctx->stream, op_ptr<const float>(a[0]), a[1], n, E,
            top, (int)a[5], op_ptr<int>(a[6]), op_ptr<float>(a[7]), op_ptr<float>(a[8]));
  GB_CHECK_LAUNCH("moe_route");
  return 1;
}

// a0 chosen experts [tokens, top], a1 tokens, a2 experts, a3 offsets [E + 1], a4 row -> pair, a5 pair -> row, a6 top
GB_OP(gb_op_moe_sort) {
  const int pairs = (int)(a[1] * a[6]), E = (int)a[2];
  if (pairs <= 0) return 0;
  if (E > MOE_MAX_EXPERTS) GB_FAIL(GB_ERR_ARG, "moe_sort: %d experts (at most %d)", E, MOE_MAX_EXPERTS);
  gb_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, ctx->stream, op_ptr<const int>(a[0]), pairs, E, op_ptr<int>(a[3]),
            op_ptr<int>(a[4]), op_ptr<int>(a[5]));
  GB_CHECK_LAUNCH("moe_sort");
  return 1;
}

// a0 h, a1 its row stride, a2 dtype (of h and rows), a3 row -> pair, a4 weights [pairs] or 0 (plain copies), a5 rows out, a6 their
// stride, a7 tokens, a8 width, a9 top
GB_OP(gb_op_moe_gather) {
  const int pairs = (int)(a[7] * a[9]), width = (int)a[8];
  if (pairs <= 0) return 0;
  const dim3 grid(pairs), block(width <= 256 ? 64 : 256);
  if (a[2] == GB_BF16)
    gb_launch(moe_gather_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const bf16>(a[0]), a[1], op_ptr<const int>(a[3]),
              op_ptr<const float>(a[4]), op_ptr<bf16>(a[5]), a[6], pairs, width, (int)a[9]);
  else
    gb_launch(moe_gather_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<const int>(a[3]),
              op_ptr<const float>(a[4]), op_ptr<float>(a[5]), a[6], pairs, width, (int)a[9]);
  GB_CHECK_LAUNCH("moe_gather");
  return 1;
}

// a0 input rows, a1 their stride, a2 their dtype, a3 weights [E, out features, in features], a4 their dtype,
// a5 offsets [E + 1], a6 experts, a7 out, a8 its row stride, a9 tokens, a10 features out (GLU: ff), a11 features in,
// a12 mode (0: GLU over [gate rows | up rows], out in the input's dtype; 1: plain, out f32), a13 top, a14 (GLU) 1 when
// gate and up rows alternate in blocks of 64 instead; f0 alpha, f1 limit, f2 what is added to u
GB_OP(gb_op_moe_experts) {
  const int pairs = (int)(a[9] * a[13]), E = (int)a[6], n_out = (int)a[10], n_in = (int)a[11], mode = (int)a[12];
  if (pairs <= 0) return 0;
  const int tiles = gb_div_up(pairs, 64) + E;            // at most this many row tiles over all experts
  const bool abf = a[2] == GB_BF16, wbf = a[4] == GB_BF16;
  if (abf && !wbf) GB_FAIL(GB_ERR_ARG, "moe_experts: bfloat16 rows with 32-bit weights");
#define GLU(TA, TW)                                                                                                 \
  gb_launch(moe_experts_glu_kernel<TA, TW>, dim3(gb_div_up(n_out, 32), tiles), dim3(256), 0, ctx->stream,          \
            op_ptr<const TA>(a[0]), a[1], op_ptr<const TW>(a[3]), op_ptr<const int>(a[5]), E, op_ptr<TA>(a[7]), a[8], \
            n_out, n_in, (float)f[0], (float)f[1], (float)f[2], (int)a[14])
#define DOWN(TA, TW)                                                                                                \
  gb_launch(moe_experts_down_kernel<TA, TW>, dim3(gb_div_up(n_out, 64), tiles), dim3(256), 0, ctx->stream,         \
            op_ptr<const TA>(a[0]), a[1], op_ptr<const TW>(a[3]), op_ptr<const int>(a[5]), E, op_ptr<float>(a[7]),   \
            a[8], n_out, n_in)
  if (mode == 0) {
    if (abf) GLU(bf16, bf16); else if (wbf) GLU(float, bf16); else GLU(float, float);
  } else {
    if (abf) DOWN(bf16, bf16); else if (wbf) DOWN(float, bf16); else DOWN(float, float);
  }
#undef GLU
#undef DOWN
  GB_CHECK_LAUNCH("moe_experts");
  return 1;
}

// a0 expert outputs by row (f32), a1 their stride, a2 pair -> row, a3 shared gate [tokens] or 0, a4 shared expert's
// output (f32) or 0, a5 its row stride, a6 y (f32), a7 its row stride, a8 tokens, a9 width, a10 top
GB_OP(gb_op_moe_combine) {
  const int n = (int)a[8], width = (int)a[9];
  if (n <= 0) return 0;
  gb_launch(moe_combine_kernel, dim3(n), dim3(width <= 256 ? 64 : 256), 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
            op_ptr<const int>(a[2]), op_ptr<const float>(a[3]), op_ptr<const float>(a[4]), a[5], op_ptr<float>(a[6]), a[7],
            width, (int)a[10]);
  GB_CHECK_LAUNCH("moe_combine");
  return 1;
}

// a0 expert outputs by row (f32), a1 their stride, a2 pair -> row, a3 chosen outputs [tokens, top], a4 their weights,
// a5 the feed-forward's input h, a6 its row stride, a7 its dtype, a8 y (f32), a9 its row stride, a10 tokens, a11 width,
// a12 top, a13 real experts (a choice from here on returns h); flags bit 0: add into y
GB_OP(gb_op_moe_combine_weighted) {
  const int n = (int)a[10], width = (int)a[11];
  if (n <= 0) return 0;
  const dim3 grid(n), block(width <= 256 ? 64 : 256);
  if (a[7] == GB_BF16)
    gb_launch(moe_combine_weighted_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
              op_ptr<const int>(a[2]), op_ptr<const int>(a[3]), op_ptr<const float>(a[4]), op_ptr<const bf16>(a[5]), a[6],
              op_ptr<float>(a[8]), a[9], width, (int)a[12], (int)a[13], flags & 1);
  else
    gb_launch(moe_combine_weighted_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
              op_ptr<const int>(a[2]), op_ptr<const int>(a[3]), op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), a[6],
              op_ptr<float>(a[8]), a[9], width, (int)a[12], (int)a[13], flags & 1);
  GB_CHECK_LAUNCH("moe_combine_weighted");
  return 1;
}
