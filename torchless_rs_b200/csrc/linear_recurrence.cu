// Gated linear recurrence with a matrix state per head (HGRN2): the forget gate also decides what
// is written.  Per head, with q, f of `dim` channels and v of `vdim` channels,
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        (S: [dim, vdim], rows belong to q's channels)
//   o_t = S_t^T q_t
//   q = silu(zq),  f = low + (1 - low) * sigmoid(zf + bias),  v = zv
// where zq, zf, zv are the 32-bit outputs of the projections.  The state is 32-bit, lives in a
// per-sequence slot, and is carried from step to step; gates, state and sums are 32-bit.
//
// The columns of S are independent of one another, so the work is spread over (sequence, head,
// group of columns); a warp owns SCAN_COLS columns, its lanes share the rows (row i = lane + 32 r),
// and the tokens of a sequence are walked in order.  One token costs a warp 2 * rows/32 * SCAN_COLS
// FMAs and SCAN_COLS warp sums; the activations of a row are computed by every warp that needs
// them rather than stored and read again.
#include "common.cuh"

#define SCAN_COLS 4          // columns per warp
#define SCAN_WARPS 4         // warps per block
#define SCAN_MAX_R 8         // rows per lane: dim <= 256

template <int R>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
gated_scan_kernel(const float* __restrict__ zq, const float* __restrict__ zf, const float* __restrict__ zv,
                  int ld, const float* __restrict__ bias, const float* __restrict__ low,
                  float* __restrict__ state, float* __restrict__ o, int ldo, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.z * SCAN_WARPS + warp) * SCAN_COLS;
  if (c0 >= vdim) return;
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * heads + h) * dim) * vdim;
  float s[R][SCAN_COLS];
  float lo[R], bi[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    lo[r] = i < dim ? low[h * dim + i] : 0.0f;
    bi[r] = i < dim ? bias[h * dim + i] : 0.0f;
#pragma unroll
    for (int c = 0; c < SCAN_COLS; ++c)
      s[r][c] = (i < dim && c0 + c < vdim) ? S[(size_t)i * vdim + c0 + c] : 0.0f;
  }
  // Tokens are taken PF at a time: their inputs are loaded and their gates computed together (all
  // independent, so the loads are in flight at once), then the state walks through them in order.
  constexpr int PF = R <= 4 ? 8 : 4;
  for (int tb = t0; tb < t1; tb += PF) {
    float qv[PF][R], fv[PF][R], vv[PF][SCAN_COLS];
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int t = tb + p < t1 ? tb + p : t1 - 1;
      const float* rq = zq + (size_t)t * ld + h * dim;
      const float* rf = zf + (size_t)t * ld + h * dim;
      const float* rv = zv + (size_t)t * ld + h * vdim + c0;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        qv[p][r] = i < dim ? rq[i] : 0.0f;
        fv[p][r] = i < dim ? rf[i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < SCAN_COLS; ++c) vv[p][c] = c0 + c < vdim ? rv[c] : 0.0f;
    }
#pragma unroll
    for (int p = 0; p < PF; ++p)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float z = qv[p][r];
        qv[p][r] = z / (1.0f + expf(-z));
        fv[p][r] = lo[r] + (1.0f - lo[r]) * (1.0f / (1.0f + expf(-(fv[p][r] + bi[r]))));
      }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float part[SCAN_COLS];
#pragma unroll
        for (int c = 0; c < SCAN_COLS; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (lane + 32 * r < dim) {
            const float f = fv[p][r], w = 1.0f - f;
#pragma unroll
            for (int c = 0; c < SCAN_COLS; ++c) {
              s[r][c] = fmaf(f, s[r][c], w * vv[p][c]);
              part[c] = fmaf(s[r][c], qv[p][r], part[c]);
            }
          }
        }
#pragma unroll
        for (int c = 0; c < SCAN_COLS; ++c) part[c] = warp_sum(part[c]);
        if (lane == 0) {
#pragma unroll
          for (int c = 0; c < SCAN_COLS; ++c)
            if (c0 + c < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + c] = part[c];
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
#pragma unroll
    for (int c = 0; c < SCAN_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// zq, zf, zv: [T, ld] 32-bit (columns of one stacked product); bias, low: [heads * dim] 32-bit;
// state: [slots, heads, dim, vdim] 32-bit; o: [T, ldo] 32-bit; B sequences, sequence b owning the
// tokens seq_start[b] .. seq_start[b + 1] - 1 of the step.
extern "C" int TL_NAME(tl_gated_scan)(const float* zq, const float* zf, const float* zv, int ld, const float* bias,
                                      const float* low, float* state, float* o, int ldo, const int* seq_start,
                                      const int* seq_slot, int B, int heads, int dim, int vdim,
                                      cudaStream_t stream) {
  if (B <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0) return TL_ERR_BAD_ARG;
  if (dim > 32 * SCAN_MAX_R || heads > 65535) return TL_ERR_UNSUPPORTED;
  const int per_block = SCAN_WARPS * SCAN_COLS;
  dim3 grid(B, heads, (vdim + per_block - 1) / per_block);
  if (grid.z > 65535) return TL_ERR_UNSUPPORTED;
  const int R = (dim + 31) / 32;
#define SCAN(RR)                                                                                        \
  return tl_launch(gated_scan_kernel<RR>, grid, dim3(SCAN_WARPS * 32), 0, stream, zq, zf, zv, ld, bias, \
                   low, state, o, ldo, seq_start, seq_slot, heads, dim, vdim)
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
}
