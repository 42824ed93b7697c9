// Gated linear attention: a matrix state per head that decays per key channel.
// Per head, with q, k, alpha of `dim` channels and v of `vdim` channels,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: [dim, vdim], rows belong to key channels)
//   o_t = S_t^T (q_t * q_scale)
//   alpha = sigmoid(za + bias)^(1 / tau) = exp(log_sigmoid(za + bias) / tau)
// where q, k, v and za are the 32-bit outputs of the projections.  The state is 32-bit, lives in a
// per-sequence slot and is carried from step to step; the decay, its logarithm, the state and all
// sums are 32-bit.
//
// The columns of S are independent of one another, so the work is spread over (sequence, head,
// group of columns); a warp owns GLA_COLS columns, its lanes share the rows (row i = lane + 32 r),
// and the tokens of a sequence are walked in order, GLA_PF at a time so that their loads and the
// transcendental work of their decays are in flight together.
#include "common.cuh"

#define GLA_COLS 4
#define GLA_WARPS 4
#define GLA_MAX_R 8          // rows per lane: states of up to 256 rows

__device__ __forceinline__ float log_sigmoid(float x) {
  // min(x, 0) - log(1 + exp(-|x|)): no overflow on either side
  return fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
}

// Lane 8 k (k = 0..3) ends with the sum over the warp of column k (6 shuffles for 4 columns).
__device__ __forceinline__ float gla_warp_sum4(const float (&part)[GLA_COLS], int lane) {
  const bool hi = lane & 16;
  float k0 = hi ? part[2] : part[0], k1 = hi ? part[3] : part[1];
  k0 += __shfl_xor_sync(0xffffffffu, hi ? part[0] : part[2], 16);
  k1 += __shfl_xor_sync(0xffffffffu, hi ? part[1] : part[3], 16);
  const bool b = lane & 8;
  float k = b ? k1 : k0;
  k += __shfl_xor_sync(0xffffffffu, b ? k0 : k1, 8);
  k += __shfl_xor_sync(0xffffffffu, k, 4);
  k += __shfl_xor_sync(0xffffffffu, k, 2);
  k += __shfl_xor_sync(0xffffffffu, k, 1);
  return k;
}

// The decays of all tokens at once, in place: za <- alpha.  For steps of many tokens per sequence,
// so that the sequential walk is left with the recurrence alone.
__global__ void gla_decay_kernel(float* __restrict__ za, int lda, const float* __restrict__ bias, float inv_tau,
                                 int T, int hd) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t total = (size_t)T * hd;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / hd;
    const int i = (int)(idx - t * hd);
    const float z = za[t * lda + i] + (bias != nullptr ? bias[i] : 0.0f);
    za[t * lda + i] = expf(log_sigmoid(z) * inv_tau);
  }
}

// PRE: `za` already holds alpha (gla_decay_kernel ran).
template <int R, bool PRE>
__global__ void __launch_bounds__(GLA_WARPS * 32)
gla_scan_kernel(const float* __restrict__ zq, const float* __restrict__ zk, const float* __restrict__ zv, int ld,
                const float* __restrict__ za, int lda, const float* __restrict__ bias, float inv_tau,
                float q_scale, float* __restrict__ state, float* __restrict__ o, int ldo,
                const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int heads, int dim,
                int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * GLA_WARPS + warp) * GLA_COLS;
  if (c0 >= vdim) return;
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * heads + h) * dim) * vdim;
  float s[R][GLA_COLS];
  float bi[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    bi[r] = (i < dim && bias != nullptr) ? bias[h * dim + i] : 0.0f;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      s[r][c] = (i < dim && c0 + c < vdim) ? S[(size_t)i * vdim + c0 + c] : 0.0f;
  }
  constexpr int PF = R <= 4 ? 8 : 4;
  for (int tb = t0; tb < t1; tb += PF) {
    float qv[PF][R], kv[PF][R], av[PF][R], vv[PF][GLA_COLS];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = tb + p < t1 ? tb + p : t1 - 1;
      const float* rq = zq + (size_t)t * ld + h * dim;
      const float* rk = zk + (size_t)t * ld + h * dim;
      const float* ra = za + (size_t)t * lda + h * dim;
      const float* rv = zv + (size_t)t * ld + h * vdim + c0;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        qv[p][r] = i < dim ? rq[i] * q_scale : 0.0f;
        kv[p][r] = i < dim ? rk[i] : 0.0f;
        av[p][r] = i < dim ? ra[i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < GLA_COLS; ++c) vv[p][c] = c0 + c < vdim ? rv[c] : 0.0f;
    }
    if (!PRE) {
#pragma unroll
      for (int p = 0; p < PF; ++p)
        if (tb + p < t1) {
#pragma unroll
          for (int r = 0; r < R; ++r) av[p][r] = expf(log_sigmoid(av[p][r] + bi[r]) * inv_tau);
        }
    }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float part[GLA_COLS];
#pragma unroll
        for (int c = 0; c < GLA_COLS; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (lane + 32 * r < dim) {
            const float a = av[p][r], k = kv[p][r];
#pragma unroll
            for (int c = 0; c < GLA_COLS; ++c) {
              s[r][c] = fmaf(a, s[r][c], k * vv[p][c]);
              part[c] = fmaf(s[r][c], qv[p][r], part[c]);
            }
          }
        }
        const float sum = gla_warp_sum4(part, lane);
        const int c = lane >> 3;
        if ((lane & 7) == 0 && c0 + c < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + c] = sum;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < GLA_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// zq, zk, zv: columns of one 32-bit product [T, ld]; za: [T, lda] 32-bit pre-activations of the decay
// (overwritten with the decays when the step has many tokens per sequence, T > 4 B); bias:
// [heads * dim] or null; state: [slots, heads, dim, vdim]; o: [T, ldo]; sequence b owns the tokens
// seq_start[b] .. seq_start[b + 1] - 1 of the step.
extern "C" int TL_NAME(tl_gla_scan)(const float* zq, const float* zk, const float* zv, int ld, float* za, int lda,
                                    const float* bias, float tau, float q_scale, float* state, float* o, int ldo,
                                    const int* seq_start, const int* seq_slot, int T, int B, int heads, int dim,
                                    int vdim, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || !(tau > 0.0f)) return TL_ERR_BAD_ARG;
  const int R = (dim + 31) / 32;
  if (heads > 65535 || R > GLA_MAX_R) return TL_ERR_UNSUPPORTED;
  const int per_block = GLA_WARPS * GLA_COLS;
  dim3 grid(B, heads, (vdim + per_block - 1) / per_block);
  if (grid.z > 65535) return TL_ERR_UNSUPPORTED;
  const float inv_tau = 1.0f / tau;
  const bool pre = T > 4 * B;
  if (pre) {
    const size_t total = (size_t)T * heads * dim;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int rc = tl_launch(gla_decay_kernel, dim3(blocks), dim3(256), 0, stream, za, lda, bias, inv_tau, T,
                             heads * dim);
    if (rc != 0) return rc;
  }
  int rc;
#define SCAN(RR)                                                                                              \
  rc = pre ? tl_launch(gla_scan_kernel<RR, true>, grid, dim3(GLA_WARPS * 32), 0, stream, zq, zk, zv, ld,      \
                       (const float*)za, lda, bias, inv_tau, q_scale, state, o, ldo, seq_start, seq_slot,     \
                       heads, dim, vdim)                                                                      \
           : tl_launch(gla_scan_kernel<RR, false>, grid, dim3(GLA_WARPS * 32), 0, stream, zq, zk, zv, ld,     \
                       (const float*)za, lda, bias, inv_tau, q_scale, state, o, ldo, seq_start, seq_slot,     \
                       heads, dim, vdim);                                                                     \
  break
  switch (R) {
    case 1: SCAN(1);
    case 2: SCAN(2);
    case 3: SCAN(3);
    case 4: SCAN(4);
    case 5: SCAN(5);
    case 6: SCAN(6);
    case 7: SCAN(7);
    default: SCAN(8);
  }
#undef SCAN
  return rc;
}
