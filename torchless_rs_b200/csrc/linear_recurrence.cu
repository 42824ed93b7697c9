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

#define SCAN_COLS 4          // columns per warp (warp_sum4 is written for 4)
#define SCAN_WARPS 4         // warps per block
#define SCAN_MAX_R 8         // rows per lane; wider states are shared out over several warps

// The gates of all tokens at once, in place: zq <- silu(zq), zf <- low + (1 - low) sigmoid(zf + bias).
// For steps of many tokens per sequence, so that the sequential walk below is left with the
// recurrence alone.
__global__ void scan_gates_kernel(float* __restrict__ zq, float* __restrict__ zf, int ld,
                                  const float* __restrict__ bias, const float* __restrict__ low, int T, int hd) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t total = (size_t)T * hd;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / hd;
    const int i = (int)(idx - t * hd);
    const float z = zq[t * ld + i];
    zq[t * ld + i] = z / (1.0f + expf(-z));
    const float l = low[i];
    zf[t * ld + i] = l + (1.0f - l) * (1.0f / (1.0f + expf(-(zf[t * ld + i] + bias[i]))));
  }
}

// Sums over the warp of SCAN_COLS (4) values per lane with 6 shuffles instead of 20: two steps hand
// half of the columns to the other half of the lanes, three more finish the one column a lane is
// left with.  Lane 8 k (k = 0..3) ends with the sum of column (k / 2) * 2 + k % 2 = k.
__device__ __forceinline__ float warp_sum4(const float (&part)[SCAN_COLS], int lane) {
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

// PRE: zq and zf already hold q and f (scan_gates_kernel ran).
template <int R, bool PRE>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
gated_scan_kernel(const float* __restrict__ zq, const float* __restrict__ zf, const float* __restrict__ zv,
                  int ld, const float* __restrict__ bias, const float* __restrict__ low,
                  float* __restrict__ state, float* __restrict__ o, int ldo, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_slot, int heads, int dim, int vdim, int row_groups, int T) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // With row_groups > 1 a warp holds the rows row0 .. row0 + 32 R - 1 only and its sums over them go to
  // slice `rg` of `o` ([row_groups][T][ldo]); scan_sum_slices_kernel adds the slices.
  const int rg = blockIdx.z % row_groups;
  const int row0 = rg * 32 * R;
  o += (size_t)rg * T * ldo;
  const int c0 = ((blockIdx.z / row_groups) * SCAN_WARPS + warp) * SCAN_COLS;
  if (c0 >= vdim) return;
  const int t0 = seq_start[b], t1 = seq_start[b + 1];
  float* S = state + (((size_t)seq_slot[b] * heads + h) * dim) * vdim;
  float s[R][SCAN_COLS];
  float lo[R], bi[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = row0 + lane + 32 * r;
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
        const int i = row0 + lane + 32 * r;
        qv[p][r] = i < dim ? rq[i] : 0.0f;
        fv[p][r] = i < dim ? rf[i] : 0.0f;
      }
#pragma unroll
      for (int c = 0; c < SCAN_COLS; ++c) vv[p][c] = c0 + c < vdim ? rv[c] : 0.0f;
    }
    if (!PRE) {
#pragma unroll
      for (int p = 0; p < PF; ++p)
        if (tb + p < t1) {
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float z = qv[p][r];
            qv[p][r] = z / (1.0f + expf(-z));
            fv[p][r] = lo[r] + (1.0f - lo[r]) * (1.0f / (1.0f + expf(-(fv[p][r] + bi[r]))));
          }
        }
    }
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      if (tb + p < t1) {
        float part[SCAN_COLS];
#pragma unroll
        for (int c = 0; c < SCAN_COLS; ++c) part[c] = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (row0 + lane + 32 * r < dim) {
            const float f = fv[p][r], w = 1.0f - f;
#pragma unroll
            for (int c = 0; c < SCAN_COLS; ++c) {
              s[r][c] = fmaf(f, s[r][c], w * vv[p][c]);
              part[c] = fmaf(s[r][c], qv[p][r], part[c]);
            }
          }
        }
        const float sum = warp_sum4(part, lane);
        const int c = lane >> 3;
        if ((lane & 7) == 0 && c0 + c < vdim) o[(size_t)(tb + p) * ldo + h * vdim + c0 + c] = sum;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = row0 + lane + 32 * r;
#pragma unroll
    for (int c = 0; c < SCAN_COLS; ++c)
      if (i < dim && c0 + c < vdim) S[(size_t)i * vdim + c0 + c] = s[r][c];
  }
}

// o[t, c] = the sum of the row groups' slices, in their order.
__global__ void scan_sum_slices_kernel(const float* __restrict__ slices, float* __restrict__ o, size_t n, int groups) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a = slices[i];
    for (int g = 1; g < groups; ++g) a += slices[(size_t)g * n + i];
    o[i] = a;
  }
}

// zq, zf, zv: [T, ld] 32-bit (columns of one stacked product); bias, low: [heads * dim] 32-bit;
// state: [slots, heads, dim, vdim] 32-bit; o: [T, ldo] 32-bit; B sequences, sequence b owning the
// tokens seq_start[b] .. seq_start[b + 1] - 1 of the step.
// `zq` and `zf` are overwritten with q and f when the step has many tokens per sequence (T > 4 B).
// `slices` (room for tl_gated_scan_groups(...) * T * ldo floats, or null): with it the rows of the state
// are shared out over that many warps per column group, for long steps (up to four times the warps to
// hide the latencies of the sequential walk) and for states of more than 256 rows; ldo must then be the
// row length of `o` (contiguous rows).
extern "C" int TL_NAME(tl_gated_scan_groups)(int T, int B, int dim) {
  const int r = (dim + 31) / 32;
  const int need = (r + SCAN_MAX_R - 1) / SCAN_MAX_R;      // a lane holds at most SCAN_MAX_R rows
  if (T <= 4 * B || T < 256) return need;
  const int fast = r >= 4 ? 4 : r >= 2 ? 2 : 1;
  return fast > need ? fast : need;
}

extern "C" int TL_NAME(tl_gated_scan)(float* zq, float* zf, const float* zv, int ld, const float* bias,
                                      const float* low, float* state, float* o, int ldo, const int* seq_start,
                                      const int* seq_slot, int T, int B, int heads, int dim, int vdim,
                                      float* slices, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0) return TL_ERR_BAD_ARG;
  if (heads > 65535) return TL_ERR_UNSUPPORTED;
  const int per_block = SCAN_WARPS * SCAN_COLS;
  const int groups = slices != nullptr ? TL_NAME(tl_gated_scan_groups)(T, B, dim) : 1;
  if (((dim + 31) / 32 + groups - 1) / groups > SCAN_MAX_R) return TL_ERR_UNSUPPORTED;   // (no slices given)
  dim3 grid(B, heads, (vdim + per_block - 1) / per_block * groups);
  if (grid.z > 65535) return TL_ERR_UNSUPPORTED;
  const int R = ((dim + 31) / 32 + groups - 1) / groups;
  float* dst = groups > 1 ? slices : o;
  const bool pre = T > 4 * B;
  if (pre) {
    const size_t total = (size_t)T * heads * dim;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int rc = tl_launch(scan_gates_kernel, dim3(blocks), dim3(256), 0, stream, zq, zf, ld, bias, low, T,
                             heads * dim);
    if (rc != 0) return rc;
  }
  int rc;
#define SCAN(RR)                                                                                               \
  rc = pre ? tl_launch(gated_scan_kernel<RR, true>, grid, dim3(SCAN_WARPS * 32), 0, stream,                    \
                       (const float*)zq, (const float*)zf, zv, ld, bias, low, state, dst, ldo, seq_start,      \
                       seq_slot, heads, dim, vdim, groups, T)                                                  \
           : tl_launch(gated_scan_kernel<RR, false>, grid, dim3(SCAN_WARPS * 32), 0, stream,                   \
                       (const float*)zq, (const float*)zf, zv, ld, bias, low, state, dst, ldo, seq_start,      \
                       seq_slot, heads, dim, vdim, groups, T);                                                 \
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
  if (rc != 0 || groups == 1) return rc;
  const size_t n = (size_t)T * ldo;
  const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  return tl_launch(scan_sum_slices_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)slices, o, n, groups);
}
