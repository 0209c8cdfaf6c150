// The gated delta rule with one decay per head and key channel, over a ragged batch of prompt portions and
// single decoded tokens, with per-request state in slots.
//
// Per head h (its queries and keys are those of key head h / (heads / kv_heads)), token after token, with
// S [dim, vdim] the head's state (32-bit, zero for a new request):
//
//     S <- diag(g_t) S                      one decay per key channel
//     u  = beta_t (v_t - S^T k_t)           what the state does not yet say about v_t
//     S <- S + k_t u^T
//     o_t = S^T q_t                         the read-out sees the token's own write
//
//  gb_op_delta_prep   what enters the recurrence, per token, all in 32-bit: q and k (after their short
//                     convolution) become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q also times
//                     q_scale; beta = sigmoid(b); g = exp(-exp(A_log[h]) * softplus(a + dt_bias))
//  gb_op_delta_scan   the recurrence; one thread owns one column of S (dim values in registers), so the two
//                     products with S are sums inside a thread and need no exchange
//
// State layout in a slot: [heads][dim][vdim].
#include "hybrid.cuh"

namespace {

// one block per token; a warp takes one key head's q or k at a time, then the threads share the rest
__global__ void delta_prep_kernel(float* qk, long long ld_qk, int k_col, const float* b, long long ld_b, float* a,
                                  long long ld_a, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                  float* beta, int H, int G, int dim, float unit_eps, float q_scale) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  for (int u = warp; u < 2 * G; u += warps) {            // u < G: a query head, else a key head
    float* x = qk + (size_t)t * ld_qk + (u < G ? u * dim : k_col + (u - G) * dim);
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss += x[d] * x[d];
    const float f = (u < G ? q_scale : 1.f) / sqrtf(warp_sum(ss) + unit_eps);
    for (int d = lane; d < dim; d += 32) x[d] *= f;
  }
  for (int i = threadIdx.x; i < H * dim; i += blockDim.x) {
    const int h = i / dim;
    float* p = a + (size_t)t * ld_a + i;
    *p = expf(-expf(a_log[h]) * hy_softplus(*p + dt_bias[i]));
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) beta[(size_t)t * H + h] = hy_sigmoid(b[(size_t)t * ld_b + h]);
}

constexpr int DS_TOKENS = 16;       // tokens whose q, k and decay are staged in shared memory at a time

// Block: (request, head, DS_COLS columns of S).  Thread j owns column c0 + j: S[i][c], i < dim, in registers
// (DK is the capacity: dim <= DK).
template <int DK, int COLS>
__global__ void __launch_bounds__(COLS)
delta_scan_kernel(const float* qk, long long ld_qk, int k_col, int v_col, const float* decay, long long ld_g,
                  const float* beta, float* state, long long slot_stride, const int* slot_ids, const int* q_start,
                  const int* q_len, float* out, long long ldo, int H, int G, int dim, int vdim) {
  extern __shared__ float staged[];                      // [3][DS_TOKENS][dim]: q, k, decay
  pdl_trigger();
  const int r = blockIdx.x, h = blockIdx.y, c = blockIdx.z * COLS + threadIdx.x;
  const int g = h / (H / G);
  const int first = q_start[r], len = q_len[r];
  const bool live = c < vdim;
  float* S = state + (size_t)slot_ids[r] * slot_stride + (size_t)h * dim * vdim + (live ? c : 0);
  float* sq = staged;
  float* sk = sq + DS_TOKENS * dim;
  float* sg = sk + DS_TOKENS * dim;
  pdl_wait();
  float s[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) s[i] = (live && i < dim) ? S[(size_t)i * vdim] : 0.f;
  for (int t0 = 0; t0 < len; t0 += DS_TOKENS) {
    const int nt = min(DS_TOKENS, len - t0);
    __syncthreads();                                     // the chunk before has been used
    for (int i = threadIdx.x; i < nt * dim; i += COLS) {
      const int tt = i / dim, d = i - tt * dim;
      const size_t row = (size_t)(first + t0 + tt);
      sq[i] = qk[row * ld_qk + g * dim + d];
      sk[i] = qk[row * ld_qk + k_col + g * dim + d];
      sg[i] = decay[row * ld_g + h * dim + d];
    }
    __syncthreads();
    if (!live) continue;
    for (int tt = 0; tt < nt; ++tt) {
      const size_t row = (size_t)(first + t0 + tt);
      const float v = qk[row * ld_qk + v_col + h * vdim + c];
      const float bt = beta[row * H + h];
      const float* q = sq + tt * dim;
      const float* k = sk + tt * dim;
      const float* gd = sg + tt * dim;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;      // four chains, added in a fixed order
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        if (i < dim) { s[i] *= gd[i]; d0 = fmaf(s[i], k[i], d0); }
        if (i + 1 < dim) { s[i + 1] *= gd[i + 1]; d1 = fmaf(s[i + 1], k[i + 1], d1); }
        if (i + 2 < dim) { s[i + 2] *= gd[i + 2]; d2 = fmaf(s[i + 2], k[i + 2], d2); }
        if (i + 3 < dim) { s[i + 3] *= gd[i + 3]; d3 = fmaf(s[i + 3], k[i + 3], d3); }
      }
      const float u = bt * (v - ((d0 + d1) + (d2 + d3)));
      d0 = d1 = d2 = d3 = 0.f;
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        if (i < dim) { s[i] = fmaf(k[i], u, s[i]); d0 = fmaf(s[i], q[i], d0); }
        if (i + 1 < dim) { s[i + 1] = fmaf(k[i + 1], u, s[i + 1]); d1 = fmaf(s[i + 1], q[i + 1], d1); }
        if (i + 2 < dim) { s[i + 2] = fmaf(k[i + 2], u, s[i + 2]); d2 = fmaf(s[i + 2], q[i + 2], d2); }
        if (i + 3 < dim) { s[i + 3] = fmaf(k[i + 3], u, s[i + 3]); d3 = fmaf(s[i + 3], q[i + 3], d3); }
      }
      out[row * ldo + h * vdim + c] = (d0 + d1) + (d2 + d3);
    }
  }
  if (!live) return;
#pragma unroll
  for (int i = 0; i < DK; ++i)
    if (i < dim) S[(size_t)i * vdim] = s[i];
}

}  // namespace

// a0 rows [q (kv_heads * dim) | k (kv_heads * dim) | v] after the convolution (f32, changed in place), a1 their
// stride, a2 column of k, a3 gate logits b [tokens, heads] (f32; a column of a wider row), a4 its row stride, a5 decay
// logits a [tokens, heads * dim] (f32, replaced by the decays), a6 its row stride, a7 dt_bias [heads * dim], a8 A_log
// [heads], a9 beta out [tokens, heads] (f32), a10 tokens, a11 heads, a12 kv heads, a13 dim; f0 what is added under the
// root of the unit norms, f1 factor on q
GB_OP(gb_op_delta_prep) {
  const int n = (int)a[10], H = (int)a[11], G = (int)a[12], dim = (int)a[13];
  if (n <= 0) return 0;
  if (G <= 0 || H % G) GB_FAIL(GB_ERR_ARG, "delta_prep: %d heads over %d key heads", H, G);
  gb_launch(delta_prep_kernel, dim3(n), dim3(256), 0, ctx->stream, op_ptr<float>(a[0]), a[1], (int)a[2],
            op_ptr<const float>(a[3]), a[4], op_ptr<float>(a[5]), a[6], op_ptr<const float>(a[7]),
            op_ptr<const float>(a[8]), op_ptr<float>(a[9]), H, G, dim, (float)f[0], (float)f[1]);
  GB_CHECK_LAUNCH("delta_prep");
  return 1;
}

// a0 rows [q | k | v] as delta_prep left them (f32), a1 their stride, a2 column of k, a3 column of v (heads * vdim),
// a4 decays [tokens, heads * dim] (f32), a5 their row stride, a6 beta [tokens, heads] (f32), a7 recurrent state of
// slot 0 ([heads][dim][vdim], f32), a8 elements between slots, a9 slot ids, a10 first row per request, a11 rows per
// request, a12 out [tokens, heads * vdim] (f32), a13 its row stride, a14 requests, a15 heads, a16 kv heads, a17 dim,
// a18 vdim
GB_OP(gb_op_delta_scan) {
  const int R = (int)a[14], H = (int)a[15], G = (int)a[16], dim = (int)a[17], vdim = (int)a[18];
  if (R <= 0) return 0;
  if (G <= 0 || H % G) GB_FAIL(GB_ERR_ARG, "delta_scan: %d heads over %d key heads", H, G);
  if (dim > 256) GB_FAIL(GB_ERR_ARG, "delta_scan: keys of %d entries (at most 256)", dim);
  const size_t smem = sizeof(float) * 3 * DS_TOKENS * (size_t)dim;
#define SCAN(DK, COLS)                                                                                                  \
  gb_launch(delta_scan_kernel<DK, COLS>, dim3(R, H, gb_div_up(vdim, COLS)), dim3(COLS), smem, ctx->stream,               \
            op_ptr<const float>(a[0]), a[1], (int)a[2], (int)a[3], op_ptr<const float>(a[4]), a[5],                      \
            op_ptr<const float>(a[6]), op_ptr<float>(a[7]), a[8], op_ptr<const int>(a[9]), op_ptr<const int>(a[10]),     \
            op_ptr<const int>(a[11]), op_ptr<float>(a[12]), a[13], H, G, dim, vdim)
  // (blocks of 32 columns where that still fills the GPU poorly: more blocks, each as fast)
  if (dim <= 32) { if (vdim <= 32) SCAN(32, 32); else SCAN(32, 64); }
  else if (dim <= 64) { if (vdim <= 32) SCAN(64, 32); else SCAN(64, 64); }
  else if (dim <= 128) SCAN(128, 32);
  else SCAN(256, 32);
#undef SCAN
  GB_CHECK_LAUNCH("delta_scan");
  return 1;
}
