// Norms over rows of the 32-bit residual stream and the small element-wise kernels around them.
//
//  gb_op_row_norm        out = norm(x[rows]) * gain, layer norm (mean taken off, variance as the mean
//                        of squared deviations) or RMS norm, statistics in 32-bit
//  gb_op_norm_add        x += norm(y) * gain: the norm AFTER a sublayer, added into the stream
//  gb_op_clamped_glu     out = g' * sigmoid(alpha g') * (u' + up_add) for rows [g | u] with clamps
//  gb_op_gelu_mul_rows   g = gelu_tanh(g) * table[id, offset : offset + dim] (a per-token input)
//  gb_op_gated_group_norm  out = rmsnorm_in_groups(y * silu(z)) * gain
//  gb_op_act_rows        out = act(x), act one of gelu (erf), gelu (tanh), silu, relu: the unit of a feed-forward
//                        without a gate; or out = act(g) * u for rows [g | u]: a gated unit
//  gb_op_scaled_sum      x += mult * (s1 * y1 + s2 * y2): two sublayers' outputs, scaled per channel, into the stream
//  gb_op_head_norm       per head: out = rmsnorm(x - lambda * x2) * gain * sigmoid(gate) * factor, each of x2,
//                        gain and gate optional: the norm behind a recurrence or behind two attention maps
#include "hybrid.cuh"

namespace {

enum { NORM_LAYER = 0, NORM_RMS = 1 };

// Rows of up to NORM_CACHE * blockDim.x values are read once and kept in registers; longer rows are read
// again from memory (an L2 hit) for every pass.
constexpr int NORM_CACHE = 8;

struct RowCache {
  float v[NORM_CACHE];
  bool whole;
};

__device__ __forceinline__ void row_load(const float* row, int dim, RowCache& c) {
  c.whole = dim <= NORM_CACHE * (int)blockDim.x;
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      c.v[i] = d < dim ? row[d] : 0.f;
    }
  }
}

// mean and 1/sqrt(var + eps) of a row of `dim` floats (the variance is the mean of the squared deviations,
// taken in a second pass); every thread of the block gets both.
__device__ __forceinline__ void row_stats(const float* row, const RowCache& c, int dim, int kind, float eps,
                                          float* scratch, float& mean, float& rstd) {
  mean = 0.f;
  if (kind == NORM_LAYER) {
    float s = 0.f;
    if (c.whole) {
#pragma unroll
      for (int i = 0; i < NORM_CACHE; ++i) s += c.v[i];
    } else {
      for (int d = threadIdx.x; d < dim; d += blockDim.x) s += row[d];
    }
    mean = block_sum(s, scratch) / (float)dim;
  }
  float ss = 0.f;
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const float v = (int)(threadIdx.x + i * blockDim.x) < dim ? c.v[i] - mean : 0.f;
      ss += v * v;
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float v = row[d] - mean;
      ss += v * v;
    }
  }
  rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
}

template <typename TO>
__global__ void row_norm_kernel(const float* x, long long ldx, const float* __restrict__ gain, TO* out, const int* rows,
                                int dim, int kind, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;                     // (the step's metadata: readable before the wait)
  pdl_wait();
  const float* row = x + (size_t)src * ldx;
  RowCache c;
  row_load(row, dim, c);
  float mean, rstd;
  row_stats(row, c, dim, kind, eps, scratch, mean, rstd);
  TO* o = out + (size_t)r * dim;
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) o[d] = from_f32<TO>((c.v[i] - mean) * rstd * gain[d]);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) o[d] = from_f32<TO>((row[d] - mean) * rstd * gain[d]);
  }
}

// x[m, :] += pend[0][m, :] + pend[1][m, :] + ... (+ bias), in this order: what a product left to be added into the
// stream, for a launch that cannot add it while it reads its rows.
__global__ void norm_pending_add_kernel(float* __restrict__ x, long long ldx, const float* pend, int splits,
                                        const float* __restrict__ bias, long long n_rows, int dim) {
  pdl_trigger();
  pdl_wait();
  const long long total = n_rows * dim;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / dim;
    const int d = (int)(i - m * dim);
    float v = x[(size_t)m * ldx + d];
    for (int u = 0; u < splits; ++u) v += pend[(size_t)u * total + i];
    if (bias) v += bias[d];
    x[(size_t)m * ldx + d] = v;
  }
}

// One warp a row, the row in registers as V4 pieces of four values a lane (dim <= 128 * V4, a multiple of 4, rows
// 16-byte aligned): no block-wide sums, 16-byte loads and packed stores.  Which kernel runs depends on the row's
// length and alignment only, never on the number of rows.
template <typename TO, int V4, bool PEND>
__global__ void __launch_bounds__(128)
row_norm_warp_kernel(const float* x, long long ldx, const float* __restrict__ gain, TO* out, const int* rows, int n, int dim,
                     int kind, float eps, const float* pend, int pend_splits, const float* __restrict__ pend_bias) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n) return;                                     // (whole warps; nothing below meets the block)
  const int src = rows ? rows[r] : r;
  pdl_wait();
  const float* row = x + (size_t)src * ldx;
  float4 v[V4];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int d = 4 * (lane + 32 * i);
    v[i] = d < dim ? *reinterpret_cast<const float4*>(row + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (PEND && d < dim) {                                 // (an instantiation of its own: the stores order the loads)
      // sums a product left to be added into the stream: added here in their order, and the row is made whole
      const size_t total = (size_t)n * dim, at = (size_t)src * dim + d;
      for (int u = 0; u < pend_splits; ++u) {
        const float4 q = *reinterpret_cast<const float4*>(pend + u * total + at);
        v[i].x += q.x; v[i].y += q.y; v[i].z += q.z; v[i].w += q.w;
      }
      if (pend_bias != nullptr) {
        const float4 q = *reinterpret_cast<const float4*>(pend_bias + d);
        v[i].x += q.x; v[i].y += q.y; v[i].z += q.z; v[i].w += q.w;
      }
      *reinterpret_cast<float4*>(const_cast<float*>(row) + d) = v[i];
    }
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = kind == NORM_LAYER ? warp_sum(s) / (float)dim : 0.f;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    if (4 * (lane + 32 * i) < dim) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      ss += (a * a + b * b) + (c * c + e * e);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int d = 4 * (lane + 32 * i);
    if (d >= dim) continue;
    const float4 g = *reinterpret_cast<const float4*>(gain + d);
    const float r0 = (v[i].x - mean) * rstd * g.x, r1 = (v[i].y - mean) * rstd * g.y;
    const float r2 = (v[i].z - mean) * rstd * g.z, r3 = (v[i].w - mean) * rstd * g.w;
    if constexpr (sizeof(TO) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
      uint2 w;
      w.x = *reinterpret_cast<unsigned*>(&lo);
      w.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(o + d) = w;
    } else {
      *reinterpret_cast<float4*>(o + d) = make_float4(r0, r1, r2, r3);
    }
  }
}

// `then`: the norm in front of the NEXT sublayer, taken of the new rows while they are in registers
// (out2 = norm2(x) * gain2), so that it needs no kernel and no second trip of its own.
struct ThenNorm {
  const float* gain;
  void* out;
  int out_dtype, kind;
  float eps;
};

__global__ void norm_add_kernel(float* x, long long ldx, const float* y, long long ldy, const float* __restrict__ gain,
                                int dim, int kind, float eps, bf16* copy, ThenNorm then) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const float* row = y + (size_t)blockIdx.x * ldy;
  float* o = x + (size_t)blockIdx.x * ldx;
  RowCache c;
  row_load(row, dim, c);
  float old[NORM_CACHE];
  if (c.whole) {                                          // the stream's own rows are requested with y's
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      old[i] = d < dim ? o[d] : 0.f;
    }
  }
  float mean, rstd;
  row_stats(row, c, dim, kind, eps, scratch, mean, rstd);
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) {
        const float v = old[i] + (c.v[i] - mean) * rstd * gain[d];
        o[d] = v;
        if (copy) copy[(size_t)blockIdx.x * dim + d] = __float2bfloat16_rn(v);
        c.v[i] = v;
      } else {
        c.v[i] = 0.f;
      }
    }
    if (then.gain != nullptr) {                         // (only with the row in registers; the host sees to that)
      float mean2, rstd2;
      row_stats(o, c, dim, then.kind, then.eps, scratch, mean2, rstd2);
#pragma unroll
      for (int i = 0; i < NORM_CACHE; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < dim) {
          const float h = (c.v[i] - mean2) * rstd2 * then.gain[d];
          if (then.out_dtype == GB_BF16) ((bf16*)then.out)[(size_t)blockIdx.x * dim + d] = __float2bfloat16_rn(h);
          else ((float*)then.out)[(size_t)blockIdx.x * dim + d] = h;
        }
      }
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float v = o[d] + (row[d] - mean) * rstd * gain[d];
      o[d] = v;
      if (copy) copy[(size_t)blockIdx.x * dim + d] = __float2bfloat16_rn(v);
    }
  }
}

// x[t, :] += mult * (s1 * y1[t, :] + s2 * y2[t, :]): the residual sum of an arrangement whose sublayers read the same
// normed rows and whose outputs are scaled channel by channel before they are added (y2, s2: optional).  `then`: the
// norm in front of the NEXT layer, taken of the new rows while they are in registers.
__global__ void scaled_sum_kernel(float* x, long long ldx, const float* y1, long long ld1, const float* __restrict__ s1,
                                  const float* y2, long long ld2, const float* __restrict__ s2, int dim, float mult,
                                  ThenNorm then) {
  __shared__ float scratch[32];
  pdl_trigger();
  float* o = x + (size_t)blockIdx.x * ldx;
  const float* a = y1 + (size_t)blockIdx.x * ld1;
  const float* b = y2 ? y2 + (size_t)blockIdx.x * ld2 : nullptr;
  pdl_wait();
  RowCache c;
  c.whole = dim <= NORM_CACHE * (int)blockDim.x;
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      float v = 0.f;
      if (d < dim) {
        float sum = s1[d] * a[d];
        if (b) sum = fmaf(s2[d], b[d], sum);
        v = fmaf(mult, sum, o[d]);
        o[d] = v;
      }
      c.v[i] = v;
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      float sum = s1[d] * a[d];
      if (b) sum = fmaf(s2[d], b[d], sum);
      o[d] = fmaf(mult, sum, o[d]);
    }
  }
  if (then.gain == nullptr) return;
  if (!c.whole) __syncthreads();                          // (the row is read again from memory)
  float mean2, rstd2;
  row_stats(o, c, dim, then.kind, then.eps, scratch, mean2, rstd2);
  if (c.whole) {
#pragma unroll
    for (int i = 0; i < NORM_CACHE; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) {
        const float h = (c.v[i] - mean2) * rstd2 * then.gain[d];
        if (then.out_dtype == GB_BF16) ((bf16*)then.out)[(size_t)blockIdx.x * dim + d] = __float2bfloat16_rn(h);
        else ((float*)then.out)[(size_t)blockIdx.x * dim + d] = h;
      }
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float h = (o[d] - mean2) * rstd2 * then.gain[d];
      if (then.out_dtype == GB_BF16) ((bf16*)then.out)[(size_t)blockIdx.x * dim + d] = __float2bfloat16_rn(h);
      else ((float*)then.out)[(size_t)blockIdx.x * dim + d] = h;
    }
  }
}

// The same with one warp a row and the row in registers as V4 pieces of four values a lane (dim <= 128 * V4, a
// multiple of 4, rows 16-byte aligned): 16-byte loads of the three rows, all in flight at once, and no block-wide
// sums.  The same arithmetic per value as above (the norm's sums are added in another order); which kernel runs
// depends on the row's length and alignment and on whether the step has 64 rows.
template <int V4>
__global__ void __launch_bounds__(128)
scaled_sum_warp_kernel(float* x, long long ldx, const float* y1, long long ld1, const float* __restrict__ s1, const float* y2,
                       long long ld2, const float* __restrict__ s2, int n, int dim, float mult, ThenNorm then) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n) return;                                     // (whole warps; nothing below meets the block)
  float* o = x + (size_t)r * ldx;
  const float* a = y1 + (size_t)r * ld1;
  const float* b = y2 ? y2 + (size_t)r * ld2 : nullptr;
  pdl_wait();
  float4 v[V4], ya[V4], yb[V4];
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int d = 4 * (lane + 32 * i);
    const bool in = d < dim;
    v[i] = in ? *reinterpret_cast<const float4*>(o + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    ya[i] = in ? *reinterpret_cast<const float4*>(a + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    yb[i] = (in && b) ? *reinterpret_cast<const float4*>(b + d) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f, sm = 0.f;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int d = 4 * (lane + 32 * i);
    if (d >= dim) continue;
    const float4 g1 = *reinterpret_cast<const float4*>(s1 + d);
    float4 sum = make_float4(g1.x * ya[i].x, g1.y * ya[i].y, g1.z * ya[i].z, g1.w * ya[i].w);
    if (b) {
      const float4 g2 = *reinterpret_cast<const float4*>(s2 + d);
      sum.x = fmaf(g2.x, yb[i].x, sum.x); sum.y = fmaf(g2.y, yb[i].y, sum.y);
      sum.z = fmaf(g2.z, yb[i].z, sum.z); sum.w = fmaf(g2.w, yb[i].w, sum.w);
    }
    v[i].x = fmaf(mult, sum.x, v[i].x); v[i].y = fmaf(mult, sum.y, v[i].y);
    v[i].z = fmaf(mult, sum.z, v[i].z); v[i].w = fmaf(mult, sum.w, v[i].w);
    *reinterpret_cast<float4*>(o + d) = v[i];
    sm += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  if (then.gain == nullptr) return;
  const float mean = then.kind == NORM_LAYER ? warp_sum(sm) / (float)dim : 0.f;
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    if (4 * (lane + 32 * i) < dim) {
      const float p = v[i].x - mean, q = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      ss += (p * p + q * q) + (c * c + e * e);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dim + then.eps);
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int d = 4 * (lane + 32 * i);
    if (d >= dim) continue;
    const float4 g = *reinterpret_cast<const float4*>(then.gain + d);
    const float r0 = (v[i].x - mean) * rstd * g.x, r1 = (v[i].y - mean) * rstd * g.y;
    const float r2 = (v[i].z - mean) * rstd * g.z, r3 = (v[i].w - mean) * rstd * g.w;
    if (then.out_dtype == GB_BF16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
      uint2 w;
      w.x = *reinterpret_cast<unsigned*>(&lo);
      w.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>((bf16*)then.out + (size_t)r * dim + d) = w;
    } else {
      *reinterpret_cast<float4*>((float*)then.out + (size_t)r * dim + d) = make_float4(r0, r1, r2, r3);
    }
  }
}

template <typename TO>
__global__ void clamped_glu_kernel(const float* gu, long long ld, TO* out, long long ldo, int n, int inner, float alpha,
                                   float limit, float up_add) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * inner) return;
  const int t = (int)(i / inner), c = (int)(i - (long long)t * inner);
  const float* row = gu + (size_t)t * ld;
  out[(size_t)t * ldo + c] = from_f32<TO>(hy_clamped_glu(row[c], row[inner + c], alpha, limit, up_add));
}

template <typename TT>
__global__ void gelu_mul_rows_kernel(float* g, long long ld, const TT* __restrict__ table, long long ldt, int offset,
                                     const int* ids, int n, int dim, int vocab, bf16* out16) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * dim) return;
  const int t = (int)(i / dim), c = (int)(i - (long long)t * dim);
  const int id = ids[t];
  const float e = (id >= 0 && id < vocab) ? to_f32(table[(size_t)id * ldt + offset + c]) : 0.f;
  float* p = g + (size_t)t * ld + c;
  const float v = hy_gelu_tanh(*p) * e;
  if (out16) out16[(size_t)t * dim + c] = __float2bfloat16_rn(v);
  else *p = v;
}

// one block per (row, group)
template <typename TO>
__global__ void gated_group_norm_kernel(const float* y, long long ldy, const float* z, long long ldz,
                                        const float* __restrict__ gain, TO* out, long long ldo, int inner, int groups,
                                        float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int width = inner / groups, c0 = g * width;
  const float* yr = y + (size_t)t * ldy + c0;
  const float* zr = z + (size_t)t * ldz + c0;
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float v = yr[d] * hy_silu(zr[d]);
    ss += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  TO* o = out + (size_t)t * ldo + c0;
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    o[d] = from_f32<TO>(yr[d] * hy_silu(zr[d]) * rstd * gain[c0 + d]);
}

enum { ACT_GELU_ERF = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU = 3 };

__device__ __forceinline__ float act_value(float z, int kind) {
  switch (kind) {
    case ACT_GELU_ERF: return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
    case ACT_GELU_TANH: return hy_gelu_tanh(z);
    case ACT_SILU: return hy_silu(z);
    default: return fmaxf(z, 0.f);
  }
}

template <typename TO>
__global__ void act_rows_kernel(const float* x, long long ld, TO* out, long long ldo, int n, int inner, int kind,
                                int up) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * inner) return;
  const int t = (int)(i / inner), c = (int)(i - (long long)t * inner);
  const float v = act_value(x[(size_t)t * ld + c], kind);
  // (`up` > 0: a gated unit whose second factor lies `up` columns further in the row)
  out[(size_t)t * ldo + c] = from_f32<TO>(up > 0 ? v * x[(size_t)t * ld + up + c] : v);
}

// Four neighbouring values a thread (rows that can be read and written in whole pieces of four); the same
// arithmetic per value as above.
template <typename TO>
__global__ void act_rows4_kernel(const float* x, long long ld, TO* out, long long ldo, int n, int inner4, int kind,
                                 int up) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * inner4) return;
  const int t = (int)(i / inner4), c = 4 * (int)(i - (long long)t * inner4);
  const float4 v = *reinterpret_cast<const float4*>(x + (size_t)t * ld + c);
  float r0 = act_value(v.x, kind), r1 = act_value(v.y, kind), r2 = act_value(v.z, kind), r3 = act_value(v.w, kind);
  if (up > 0) {
    const float4 u = *reinterpret_cast<const float4*>(x + (size_t)t * ld + up + c);
    r0 *= u.x; r1 *= u.y; r2 *= u.z; r3 *= u.w;
  }
  TO* o = out + (size_t)t * ldo + c;
  if constexpr (sizeof(TO) == 2) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
    uint2 w;
    w.x = *reinterpret_cast<unsigned*>(&lo);
    w.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(o) = w;
  } else {
    *reinterpret_cast<float4*>(o) = make_float4(r0, r1, r2, r3);
  }
}

// one warp per (row, head); values of up to 32 * HN_VR entries stay in registers
constexpr int HN_VR = 8;

template <typename TO>
__global__ void head_norm_kernel(const float* x, long long ldx, long long xh, const float* x2,
                                 const float* __restrict__ gain, const float* gate, long long ld_gate, TO* out,
                                 long long ldo, int n, int H, int vdim, float eps, float lambda, float factor) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= (long long)n * H) return;
  const int t = (int)(idx / H), h = (int)(idx - (long long)t * H);
  const size_t at = (size_t)t * ldx + (size_t)h * xh;
  float v[HN_VR];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < HN_VR; ++i) {
    const int d = lane + 32 * i;
    v[i] = 0.f;
    if (d < vdim) v[i] = x2 ? x[at + d] - lambda * x2[at + d] : x[at + d];
    ss += v[i] * v[i];
  }
  const float rstd = factor / sqrtf(warp_sum(ss) / (float)vdim + eps);
#pragma unroll
  for (int i = 0; i < HN_VR; ++i) {
    const int d = lane + 32 * i;
    if (d >= vdim) continue;
    float o = v[i] * rstd;
    if (gain) o *= gain[d];
    if (gate) o *= hy_sigmoid(gate[(size_t)t * ld_gate + (size_t)h * vdim + d]);
    out[(size_t)t * ldo + (size_t)h * vdim + d] = from_f32<TO>(o);
  }
}

inline int norm_threads(int dim) { return dim <= 256 ? 64 : dim <= 1024 ? 128 : 256; }

}  // namespace

// a0 x (f32), a1 its row stride, a2 gain, a3 out [rows, dim], a4 out dtype, a5 row list (int32) or 0, a6 rows,
// a7 dim, a8 kind (0 layer norm, 1 RMS norm); f0 eps
GB_OP(gb_op_row_norm) {
  const int n = (int)a[6], dim = (int)a[7], kind = (int)a[8];
  if (n <= 0) return 0;
  if (kind != NORM_LAYER && kind != NORM_RMS) GB_FAIL(GB_ERR_ARG, "row_norm: kind %d", kind);
  const size_t out_bytes = a[4] == GB_BF16 ? 2 : 4;
  const bool by_warps = dim % 4 == 0 && dim <= 2048 && a[1] % 4 == 0 && (a[0] & 15) == 0 && (a[2] & 15) == 0 &&
                        (a[3] & (4 * out_bytes - 1)) == 0;
  // sums a product left to be added into the stream (a record with GB_OP_TAKES_PENDING): the kernel with a warp a row
  // adds them while it reads its rows, when these are all of the stream's rows; else they are added first
  const float* pend = (flags & GB_OP_TAKES_PENDING) && ctx->pend_splits > 0 ? ctx->pend : nullptr;
  int launched = 0;
  if (pend != nullptr) {
    const long long N = ctx->sym != nullptr ? ctx->sym[GB_SYM_TOKENS] : n;
    const bool folds = by_warps && a[5] == 0 && op_ptr<float>(a[0]) == ctx->residual && a[1] == ctx->residual_ld &&
                       dim == ctx->residual_ld && n == N && ((uintptr_t)pend & 15) == 0 &&
                       (ctx->pend_bias == nullptr || ((uintptr_t)ctx->pend_bias & 15) == 0);
    if (!folds) {
      const long long total = N * ctx->residual_ld;
      const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
      gb_launch(norm_pending_add_kernel, dim3(blocks), dim3(256), 0, ctx->stream, ctx->residual, ctx->residual_ld, pend,
                ctx->pend_splits, ctx->pend_bias, N, (int)ctx->residual_ld);
      GB_CHECK_LAUNCH("row_norm (pending sums)");
      pend = nullptr;
      launched = 1;
    }
  }
  if (by_warps) {
    const dim3 wgrid(gb_div_up(n, 4)), wblock(128);
#define WARP_NORM(TO, V4)                                                                                               \
    if (pend != nullptr)                                                                                                \
      gb_launch(row_norm_warp_kernel<TO, V4, true>, wgrid, wblock, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],      \
                op_ptr<const float>(a[2]), op_ptr<TO>(a[3]), op_ptr<const int>(a[5]), n, dim, kind, (float)f[0], pend,    \
                ctx->pend_splits, ctx->pend_bias);                                                                       \
    else                                                                                                                \
    gb_launch(row_norm_warp_kernel<TO, V4, false>, wgrid, wblock, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],       \
              op_ptr<const float>(a[2]), op_ptr<TO>(a[3]), op_ptr<const int>(a[5]), n, dim, kind, (float)f[0], pend,          \
              pend != nullptr ? ctx->pend_splits : 0, pend != nullptr ? ctx->pend_bias : nullptr)
#define WARP_NORM_V4(TO)                                                                                                \
    do {                                                                                                                \
      if (dim <= 128) WARP_NORM(TO, 1); else if (dim <= 256) WARP_NORM(TO, 2); else if (dim <= 512) WARP_NORM(TO, 4);   \
      else if (dim <= 1024) WARP_NORM(TO, 8); else WARP_NORM(TO, 16);                                                   \
    } while (0)
    if (a[4] == GB_BF16) WARP_NORM_V4(bf16); else WARP_NORM_V4(float);
#undef WARP_NORM_V4
#undef WARP_NORM
    GB_CHECK_LAUNCH("row_norm (a warp a row)");
    return launched + 1;
  }
  const dim3 grid(n), block(norm_threads(dim));
  if (a[4] == GB_BF16)
    gb_launch(row_norm_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<const float>(a[2]),
              op_ptr<bf16>(a[3]), op_ptr<const int>(a[5]), dim, kind, (float)f[0]);
  else
    gb_launch(row_norm_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<const float>(a[2]),
              op_ptr<float>(a[3]), op_ptr<const int>(a[5]), dim, kind, (float)f[0]);
  GB_CHECK_LAUNCH("row_norm");
  return launched + 1;
}

// a0 x (f32, the stream), a1 its row stride, a2 y (f32), a3 its row stride, a4 gain, a5 rows, a6 dim, a7 kind,
// a8 a bfloat16 copy of the new rows [rows, dim] for a product that reads the stream next, or 0; a9 gain of a second
// norm, taken of the new rows (the norm in front of the next sublayer), or 0; a10 its output [rows, dim], a11 the
// output's dtype, a12 its kind; f0 eps, f1 the second norm's eps
GB_OP(gb_op_norm_add) {
  const int n = (int)a[5], dim = (int)a[6], kind = (int)a[7];
  if (n <= 0) return 0;
  if (kind != NORM_LAYER && kind != NORM_RMS) GB_FAIL(GB_ERR_ARG, "norm_add: kind %d", kind);
  const int threads = norm_threads(dim);
  ThenNorm then = {op_ptr<const float>(a[9]), op_ptr<void>(a[10]), (int)a[11], (int)a[12], (float)f[1]};
  const bool second = then.gain != nullptr;
  if (second && then.kind != NORM_LAYER && then.kind != NORM_RMS) GB_FAIL(GB_ERR_ARG, "norm_add: second kind %d", then.kind);
  const bool fused = second && dim <= NORM_CACHE * threads;   // the row fits the registers
  ThenNorm none = {nullptr, nullptr, 0, 0, 0.f};
  gb_launch(norm_add_kernel, dim3(n), dim3(threads), 0, ctx->stream, op_ptr<float>(a[0]), a[1],
            op_ptr<const float>(a[2]), a[3], op_ptr<const float>(a[4]), dim, kind, (float)f[0], op_ptr<bf16>(a[8]),
            fused ? then : none);
  GB_CHECK_LAUNCH("norm_add");
  if (!second || fused) return 1;
  // a row too long for the registers: the second norm as a kernel of its own
  if (then.out_dtype == GB_BF16)
    gb_launch(row_norm_kernel<bf16>, dim3(n), dim3(threads), 0, ctx->stream, op_ptr<const float>(a[0]), a[1], then.gain,
              (bf16*)then.out, (const int*)nullptr, dim, then.kind, then.eps);
  else
    gb_launch(row_norm_kernel<float>, dim3(n), dim3(threads), 0, ctx->stream, op_ptr<const float>(a[0]), a[1], then.gain,
              (float*)then.out, (const int*)nullptr, dim, then.kind, then.eps);
  GB_CHECK_LAUNCH("norm_add (second norm)");
  return 2;
}

// a0 rows [g | u] (f32), a1 their stride, a2 out [n, inner], a3 out dtype, a4 its row stride, a5 rows, a6 inner;
// f0 alpha, f1 limit, f2 what is added to u
GB_OP(gb_op_clamped_glu) {
  const int n = (int)a[5], inner = (int)a[6];
  if (n <= 0) return 0;
  const dim3 grid(gb_div_up((long long)n * inner, 256)), block(256);
  if (a[3] == GB_BF16)
    gb_launch(clamped_glu_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<bf16>(a[2]),
              a[4], n, inner, (float)f[0], (float)f[1], (float)f[2]);
  else
    gb_launch(clamped_glu_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<float>(a[2]),
              a[4], n, inner, (float)f[0], (float)f[1], (float)f[2]);
  GB_CHECK_LAUNCH("clamped_glu");
  return 1;
}

// a0 g (f32, in place), a1 its row stride, a2 table, a3 its dtype, a4 its row stride, a5 first column, a6 token ids,
// a7 rows, a8 dim, a9 rows of the table, a10 a bfloat16 output [rows, dim] instead of writing in place, or 0
GB_OP(gb_op_gelu_mul_rows) {
  const int n = (int)a[7], dim = (int)a[8];
  if (n <= 0) return 0;
  const dim3 grid(gb_div_up((long long)n * dim, 256)), block(256);
  if (a[3] == GB_BF16)
    gb_launch(gelu_mul_rows_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<float>(a[0]), a[1], op_ptr<const bf16>(a[2]),
              a[4], (int)a[5], op_ptr<const int>(a[6]), n, dim, (int)a[9], op_ptr<bf16>(a[10]));
  else
    gb_launch(gelu_mul_rows_kernel<float>, grid, block, 0, ctx->stream, op_ptr<float>(a[0]), a[1], op_ptr<const float>(a[2]),
              a[4], (int)a[5], op_ptr<const int>(a[6]), n, dim, (int)a[9], op_ptr<bf16>(a[10]));
  GB_CHECK_LAUNCH("gelu_mul_rows");
  return 1;
}

// a0 y (f32), a1 its row stride, a2 z (f32), a3 its row stride, a4 gain [inner], a5 out, a6 out dtype, a7 its row
// stride, a8 rows, a9 inner, a10 groups; f0 eps
GB_OP(gb_op_gated_group_norm) {
  const int n = (int)a[8], inner = (int)a[9], groups = (int)a[10];
  if (n <= 0) return 0;
  if (groups <= 0 || inner % groups) GB_FAIL(GB_ERR_ARG, "gated_group_norm: %d columns in %d groups", inner, groups);
  const dim3 grid(n, groups), block(norm_threads(inner / groups));
  if (a[6] == GB_BF16)
    gb_launch(gated_group_norm_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
              op_ptr<const float>(a[2]), a[3], op_ptr<const float>(a[4]), op_ptr<bf16>(a[5]), a[7], inner, groups, (float)f[0]);
  else
    gb_launch(gated_group_norm_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
              op_ptr<const float>(a[2]), a[3], op_ptr<const float>(a[4]), op_ptr<float>(a[5]), a[7], inner, groups, (float)f[0]);
  GB_CHECK_LAUNCH("gated_group_norm");
  return 1;
}

// a0 x (f32, the stream), a1 its row stride, a2 y1 (f32), a3 its row stride, a4 s1 [dim] (f32), a5 y2 (f32) or 0, a6 its
// row stride, a7 s2 [dim] (f32), a8 rows, a9 dim; optionally the norm in front of the next layer, taken of the new rows:
// a10 its gain (0: none), a11 out [rows, dim], a12 out dtype, a13 kind; f0 the factor on the sum, f1 that norm's eps
GB_OP(gb_op_scaled_sum) {
  const int n = (int)a[8], dim = (int)a[9];
  if (n <= 0) return 0;
  if (a[5] && !a[7]) GB_FAIL(GB_ERR_ARG, "scaled_sum: a second branch without its scale");
  ThenNorm then{op_ptr<const float>(a[10]), op_ptr<void>(a[11]), (int)a[12], (int)a[13], (float)f[1]};
  const long long out_align = a[12] == GB_BF16 ? 7 : 15;
  // (a warp a row pays with 64 rows and more, and while the three rows' pieces fit a lane's registers: measured 16 against
  // 19 µs for 2,048 rows of 1,024, but 30 against 28 µs at 2,048 entries, and 23 against 14 µs for a decode step's 8 rows)
  const bool by_warps = n >= 64 && dim % 4 == 0 && dim <= 1024 && a[1] % 4 == 0 && a[3] % 4 == 0 && (a[0] & 15) == 0 && (a[2] & 15) == 0 &&
                        (a[4] & 15) == 0 && (!a[5] || (a[6] % 4 == 0 && (a[5] & 15) == 0 && (a[7] & 15) == 0)) &&
                        (!a[10] || ((a[10] & 15) == 0 && (a[11] & out_align) == 0));
  if (by_warps) {
    const dim3 wgrid(gb_div_up(n, 4)), wblock(128);
#define SUM_WARP(V4)                                                                                                    \
    gb_launch(scaled_sum_warp_kernel<V4>, wgrid, wblock, 0, ctx->stream, op_ptr<float>(a[0]), a[1],                      \
              op_ptr<const float>(a[2]), a[3], op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), a[6],               \
              op_ptr<const float>(a[7]), n, dim, (float)f[0], then)
    if (dim <= 128) SUM_WARP(1); else if (dim <= 256) SUM_WARP(2); else if (dim <= 512) SUM_WARP(4);
    else SUM_WARP(8);
#undef SUM_WARP
    GB_CHECK_LAUNCH("scaled_sum (a warp a row)");
    return 1;
  }
  const dim3 block(dim >= 2048 ? 512 : dim > 512 ? 256 : 128);
  gb_launch(scaled_sum_kernel, dim3(n), block, 0, ctx->stream, op_ptr<float>(a[0]), a[1], op_ptr<const float>(a[2]), a[3],
            op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), a[6], op_ptr<const float>(a[7]), dim, (float)f[0], then);
  GB_CHECK_LAUNCH("scaled_sum");
  return 1;
}

// a0 x (f32), a1 its row stride, a2 out [rows, inner], a3 out dtype, a4 its row stride, a5 rows, a6 inner, a7 which
// function: 0 gelu (erf), 1 gelu (tanh), 2 silu, 3 relu, a8 gated (0/1): the rows are [g | u] of `inner` entries each
// and out = act(g) * u
GB_OP(gb_op_act_rows) {
  const int n = (int)a[5], inner = (int)a[6];
  const int up = a[8] ? inner : 0;
  if (n <= 0) return 0;
  if (a[7] > ACT_RELU) GB_FAIL(GB_ERR_ARG, "act_rows: function %lld", a[7]);
  const size_t out_bytes = a[3] == GB_BF16 ? 2 : 4;
  if (inner % 4 == 0 && a[1] % 4 == 0 && a[4] % 4 == 0 && (a[0] & 15) == 0 && (a[2] & (4 * out_bytes - 1)) == 0) {
    const dim3 grid4(gb_div_up((long long)n * (inner / 4), 256)), block4(256);
    if (a[3] == GB_BF16)
      gb_launch(act_rows4_kernel<bf16>, grid4, block4, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<bf16>(a[2]),
                a[4], n, inner / 4, (int)a[7], up);
    else
      gb_launch(act_rows4_kernel<float>, grid4, block4, 0, ctx->stream, op_ptr<const float>(a[0]), a[1],
                op_ptr<float>(a[2]), a[4], n, inner / 4, (int)a[7], up);
    GB_CHECK_LAUNCH("act_rows (four a thread)");
    return 1;
  }
  const dim3 grid(gb_div_up((long long)n * inner, 256)), block(256);
  if (a[3] == GB_BF16)
    gb_launch(act_rows_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<bf16>(a[2]), a[4],
              n, inner, (int)a[7], up);
  else
    gb_launch(act_rows_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], op_ptr<float>(a[2]),
              a[4], n, inner, (int)a[7], up);
  GB_CHECK_LAUNCH("act_rows");
  return 1;
}

// a0 x (f32; head h of row t starts at t * a1 + h * a2), a1 row stride, a2 elements between heads, a3 x2 (f32, laid
// out as x) or 0, a4 gain [vdim] (shared by the heads) or 0, a5 gate logits (f32, [t, h * vdim + d] at a row stride)
// or 0, a6 that stride, a7 out [rows, heads * vdim], a8 out dtype, a9 its row stride, a10 rows, a11 heads, a12 vdim;
// f0 eps, f1 lambda, f2 factor
GB_OP(gb_op_head_norm) {
  const int n = (int)a[10], H = (int)a[11], vdim = (int)a[12];
  if (n <= 0) return 0;
  if (vdim > 32 * HN_VR) GB_FAIL(GB_ERR_ARG, "head_norm: heads of %d values (at most %d)", vdim, 32 * HN_VR);
  const dim3 grid(gb_div_up((long long)n * H, 4)), block(128);
  if (a[8] == GB_BF16)
    gb_launch(head_norm_kernel<bf16>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], a[2],
              op_ptr<const float>(a[3]), op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), a[6], op_ptr<bf16>(a[7]), a[9],
              n, H, vdim, (float)f[0], (float)f[1], (float)f[2]);
  else
    gb_launch(head_norm_kernel<float>, grid, block, 0, ctx->stream, op_ptr<const float>(a[0]), a[1], a[2],
              op_ptr<const float>(a[3]), op_ptr<const float>(a[4]), op_ptr<const float>(a[5]), a[6], op_ptr<float>(a[7]), a[9],
              n, H, vdim, (float)f[0], (float)f[1], (float)f[2]);
  GB_CHECK_LAUNCH("head_norm");
  return 1;
}
