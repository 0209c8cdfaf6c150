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
//  gb_op_delta_scan   the recurrence; a column of S (dim values) lives in the registers of one thread, or,
//                     where rows can be copied in 16-byte pieces, of up to 16 neighbouring lanes that add
//                     their shares of the two products with S by shuffles
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

// The same recurrence with a column of S shared by SPLIT neighbouring lanes, each with PER of the column's dim
// values (dim <= SPLIT * PER), so a token costs a thread 4 PER operations and the column 2 log2(SPLIT) shuffles;
// q, k and the decays are read from shared memory four values an instruction.  The inputs of TOK tokens at a
// time (q, k, decay, the block's columns of v, beta) arrive by asynchronous copies into one of two buffers
// while the tokens of the other are consumed, so the recurrence itself reads nothing from global memory.
// The sums over dim run in another order than in the kernel above; which of the two runs depends on the
// layer's sizes only.
constexpr int DCOL_THREADS = 64;

__device__ __forceinline__ void dcol_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void dcol_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}

template <int SPLIT, int PER, int TOK>
__global__ void __launch_bounds__(DCOL_THREADS)
delta_scan_cols_kernel(const float* qk, long long ld_qk, int k_col, int v_col, const float* decay, long long ld_g,
                       const float* beta, float* state, long long slot_stride, const int* slot_ids, const int* q_start,
                       const int* q_len, float* out, long long ldo, int H, int G, int dim, int vdim) {
  constexpr int NR = SPLIT * PER, COLS = DCOL_THREADS / SPLIT, Q4 = PER / 4;
  constexpr int BUF = TOK * (3 * NR + COLS) + ((TOK + 3) & ~3);   // q [TOK][NR] | k | decay | v [TOK][COLS] | beta [TOK]
  extern __shared__ __align__(16) float dcol[];                   // [2][BUF]
  pdl_trigger();
  const int col = threadIdx.x / SPLIT, q = threadIdx.x % SPLIT;
  const int r = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS, c = c0 + col;
  const bool active = c < vdim;
  const int g = h / (H / G);
  const int first = q_start[r], len = q_len[r];
  float* S = state + (size_t)slot_ids[r] * slot_stride + (size_t)h * dim * vdim + (active ? c : 0);
  if (dim < NR)                                                   // the padding dim .. NR of q, k and decay stays zero
    for (int i = threadIdx.x; i < 2 * BUF; i += DCOL_THREADS) dcol[i] = 0.f;
  pdl_wait();
  // this thread's rows of the column: n = 4 (q + SPLIT i) + e, i < Q4, e < 4
  float s[PER];
#pragma unroll
  for (int i = 0; i < Q4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = 4 * (q + SPLIT * i) + e;
      s[4 * i + e] = (active && n < dim) ? S[(size_t)n * vdim] : 0.f;
    }
  __syncthreads();

  // What a thread copies is the same for every token: 16-byte piece number threadIdx.x (+ 64, ...) of a token's
  // [q | k | decay | this block's columns of v]; source, row stride and place in the buffer are worked out once.
  const int pieces = dim >> 2, vpieces = min(COLS, vdim - c0) >> 2;
  constexpr int ROLES = (3 * NR / 4 + COLS / 4 + DCOL_THREADS - 1) / DCOL_THREADS;
  const float* r_src[ROLES];
  long long r_ld[ROLES];
  int r_dst[ROLES], r_step[ROLES];
#pragma unroll
  for (int j = 0; j < ROLES; ++j) {
    const int i = threadIdx.x + j * DCOL_THREADS;
    r_src[j] = nullptr;
    r_ld[j] = 0;
    r_dst[j] = r_step[j] = 0;
    if (i < 3 * pieces) {
      const int which = i / pieces, c4 = i - which * pieces;
      r_src[j] = which == 2 ? decay + (size_t)first * ld_g + h * dim + 4 * c4
                            : qk + (size_t)first * ld_qk + (which ? k_col : 0) + g * dim + 4 * c4;
      r_ld[j] = which == 2 ? ld_g : ld_qk;
      r_dst[j] = which * TOK * NR + 4 * c4;
      r_step[j] = NR;
    } else if (i < 3 * pieces + vpieces) {
      const int c4 = i - 3 * pieces;
      r_src[j] = qk + (size_t)first * ld_qk + v_col + h * vdim + c0 + 4 * c4;
      r_ld[j] = ld_qk;
      r_dst[j] = 3 * TOK * NR + 4 * c4;
      r_step[j] = COLS;
    }
  }
  auto stage = [&](int t0, int b) {
    const int nt = min(TOK, len - t0);
    float* Q = dcol + b * BUF;
    float* V = Q + 3 * TOK * NR;
    for (int tt = 0; tt < nt; ++tt) {
#pragma unroll
      for (int j = 0; j < ROLES; ++j)
        if (r_src[j]) gb_cp_async_16(Q + r_dst[j] + tt * r_step[j], r_src[j] + (size_t)(t0 + tt) * r_ld[j]);
    }
    if ((int)threadIdx.x < nt)
      gb_cp_async_4(V + TOK * COLS + threadIdx.x, beta + (size_t)(first + t0 + threadIdx.x) * H + h);
    dcol_commit();
  };

  if (len > 0) stage(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < len; t0 += TOK, b ^= 1) {
    const int nt = min(TOK, len - t0);
    if (t0 + TOK < len) {
      stage(t0 + TOK, b ^ 1);
      dcol_wait<1>();                                             // this chunk has landed, the next is on its way
    } else {
      dcol_wait<0>();
    }
    __syncthreads();
    const float* Q = dcol + b * BUF;
    const float* K = Q + TOK * NR;
    const float* Gd = K + TOK * NR;
    const float* V = Gd + TOK * NR;
    const float* Bt = V + TOK * COLS;
    // A warp issues in order and is alone on its scheduler, so what does not depend on the token's chain is
    // placed where the chain waits: token tt + 1's operands are read from shared memory while token tt is
    // computed, and token tt's read-out is summed over the lanes and stored while token tt + 1's chain runs.
    float4 g4[Q4], k4[Q4], q4[Q4];
#pragma unroll
    for (int i = 0; i < Q4; ++i) {
      g4[i] = *reinterpret_cast<const float4*>(Gd + 4 * (q + SPLIT * i));
      k4[i] = *reinterpret_cast<const float4*>(K + 4 * (q + SPLIT * i));
      q4[i] = *reinterpret_cast<const float4*>(Q + 4 * (q + SPLIT * i));
    }
    float v = active ? V[col] : 0.f, bt = Bt[0];
    float o_before = 0.f;                                         // token tt - 1's read-out, this lane's share
#pragma unroll 2
    for (int tt = 0; tt < nt; ++tt) {                             // (every lane, also of a column beyond vdim: the shuffles)
      const int tn = min(tt + 1, nt - 1);
      float4 g4n[Q4], k4n[Q4], q4n[Q4];
#pragma unroll
      for (int i = 0; i < Q4; ++i) {
        g4n[i] = *reinterpret_cast<const float4*>(Gd + tn * NR + 4 * (q + SPLIT * i));
        k4n[i] = *reinterpret_cast<const float4*>(K + tn * NR + 4 * (q + SPLIT * i));
        q4n[i] = *reinterpret_cast<const float4*>(Q + tn * NR + 4 * (q + SPLIT * i));
      }
      const float vn = active ? V[tn * COLS + col] : 0.f, btn = Bt[tn];
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;               // four chains, added in a fixed order
#pragma unroll
      for (int i = 0; i < Q4; ++i) {
        s[4 * i] *= g4[i].x;         d0 = fmaf(s[4 * i], k4[i].x, d0);
        s[4 * i + 1] *= g4[i].y;     d1 = fmaf(s[4 * i + 1], k4[i].y, d1);
        s[4 * i + 2] *= g4[i].z;     d2 = fmaf(s[4 * i + 2], k4[i].z, d2);
        s[4 * i + 3] *= g4[i].w;     d3 = fmaf(s[4 * i + 3], k4[i].w, d3);
      }
      float dot = (d0 + d1) + (d2 + d3);
      float ob = o_before;
#pragma unroll
      for (int w = 1; w < SPLIT; w <<= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, w);
        ob += __shfl_xor_sync(0xffffffffu, ob, w);
      }
      if (active && q == 0 && tt > 0) out[(size_t)(first + t0 + tt - 1) * ldo + h * vdim + c] = ob;
      const float u = bt * (v - dot);
      d0 = d1 = d2 = d3 = 0.f;
#pragma unroll
      for (int i = 0; i < Q4; ++i) {
        s[4 * i] = fmaf(k4[i].x, u, s[4 * i]);             d0 = fmaf(s[4 * i], q4[i].x, d0);
        s[4 * i + 1] = fmaf(k4[i].y, u, s[4 * i + 1]);     d1 = fmaf(s[4 * i + 1], q4[i].y, d1);
        s[4 * i + 2] = fmaf(k4[i].z, u, s[4 * i + 2]);     d2 = fmaf(s[4 * i + 2], q4[i].z, d2);
        s[4 * i + 3] = fmaf(k4[i].w, u, s[4 * i + 3]);     d3 = fmaf(s[4 * i + 3], q4[i].w, d3);
      }
      o_before = (d0 + d1) + (d2 + d3);
#pragma unroll
      for (int i = 0; i < Q4; ++i) { g4[i] = g4n[i]; k4[i] = k4n[i]; q4[i] = q4n[i]; }
      v = vn;
      bt = btn;
    }
#pragma unroll
    for (int w = 1; w < SPLIT; w <<= 1) o_before += __shfl_xor_sync(0xffffffffu, o_before, w);
    if (active && q == 0) out[(size_t)(first + t0 + nt - 1) * ldo + h * vdim + c] = o_before;
    __syncthreads();                                              // before the copies of the chunk after next land here
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < Q4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = 4 * (q + SPLIT * i) + e;
        if (n < dim) S[(size_t)n * vdim] = s[4 * i + e];
      }
  }
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
// a18 vdim; flags bit 0: the kernel with one thread a column, whatever the sizes
GB_OP(gb_op_delta_scan) {
  const int R = (int)a[14], H = (int)a[15], G = (int)a[16], dim = (int)a[17], vdim = (int)a[18];
  if (R <= 0) return 0;
  if (G <= 0 || H % G) GB_FAIL(GB_ERR_ARG, "delta_scan: %d heads over %d key heads", H, G);
  if (dim > 256) GB_FAIL(GB_ERR_ARG, "delta_scan: keys of %d entries (at most 256)", dim);
  // rows that can be copied in 16-byte pieces: a column of S over several lanes, inputs staged ahead
  if (!(flags & 1) && dim % 4 == 0 && vdim % 4 == 0 && a[1] % 4 == 0 && a[2] % 4 == 0 && a[3] % 4 == 0 && a[5] % 4 == 0 &&
      (a[0] & 15) == 0 && (a[4] & 15) == 0) {
#define COLS_SCAN(SPLIT, PER, TOK)                                                                                      \
    gb_launch(delta_scan_cols_kernel<SPLIT, PER, TOK>, dim3(R, H, gb_div_up(vdim, DCOL_THREADS / SPLIT)),                \
              dim3(DCOL_THREADS),                                                                                       \
              sizeof(float) * 2 * ((size_t)TOK * (3 * SPLIT * PER + DCOL_THREADS / SPLIT) + ((TOK + 3) & ~3)),          \
              ctx->stream, op_ptr<const float>(a[0]), a[1], (int)a[2], (int)a[3], op_ptr<const float>(a[4]), a[5],       \
              op_ptr<const float>(a[6]), op_ptr<float>(a[7]), a[8], op_ptr<const int>(a[9]), op_ptr<const int>(a[10]),   \
              op_ptr<const int>(a[11]), op_ptr<float>(a[12]), a[13], H, G, dim, vdim)
    if (dim <= 8) COLS_SCAN(1, 8, 16);
    else if (dim <= 16) COLS_SCAN(2, 8, 16);
    else if (dim <= 32) COLS_SCAN(4, 8, 16);
    else if (dim <= 64) COLS_SCAN(8, 8, 16);
    else if (dim <= 128) COLS_SCAN(8, 16, 8);
    else COLS_SCAN(16, 16, 4);
#undef COLS_SCAN
    GB_CHECK_LAUNCH("delta_scan (columns)");
    return 1;
  }
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
