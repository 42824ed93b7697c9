// Memory-bound kernels of arrangements whose sublayers read the 32-bit stream itself and whose
// outputs are normalised before they join it:
//   - an embedding addend chosen by a hash of (previous token, token), with the previous token
//     of every sequence kept as per-sequence state;
//   - x += m * g * y / rms(y) with a single gain g (the norm sits on the branch's output), which
//     also writes the activation-type copy of the new stream that the next products read;
//   - the polynomial activation of normalised powers of a feed-forward.
// Sums of squares, roots and the stream are 32-bit in both builds.
#include "common.cuh"

// Token t of the step: from the host's array, or from the tokens that the previous step selected.
__device__ __forceinline__ int step_token(const int* tokens, const int* token_from, const int* token_src,
                                          int t, int vocab) {
  int tok = tokens[t];
  if (token_src != nullptr && token_from[t] >= 0) tok = token_src[token_from[t]];
  return tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
}

// ---------------------------------------------------------------------------
// x[t, :] += table[row, :], row = (prev * mul_prev + tok * mul_cur) mod buckets, and row =
// buckets (the table's last row) for a sequence's first token.  `prev` is the token before in
// this step, or, for the first token that a sequence brings to this step, what `last_token`
// holds for the sequence's slot.  This kernel only reads `last_token`; remember_last_token_kernel
// writes it afterwards (a block here may run after the block of the sequence's last token).
// ---------------------------------------------------------------------------
__global__ void pair_embed_add_kernel(const int* __restrict__ tokens, const int* __restrict__ token_from,
                                      const int* __restrict__ token_src, const int* __restrict__ token_pos,
                                      const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                      const int* __restrict__ seq_start, const int* __restrict__ last_token,
                                      const act_t* __restrict__ table, float* __restrict__ x, int H, int vocab,
                                      int buckets, long long mul_prev, long long mul_cur) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  long long row = buckets;
  if (token_pos[t] > 0) {
    const int s = token_seq[t];
    const long long tok = step_token(tokens, token_from, token_src, t, vocab);
    const long long prev = t == seq_start[s] ? (long long)last_token[seq_slot[s]]
                                             : (long long)step_token(tokens, token_from, token_src, t - 1, vocab);
    row = (prev * mul_prev + tok * mul_cur) % (long long)buckets;
    if (row < 0) row += buckets;
  }
  const act_t* src = table + (size_t)row * H;
  float* dst = x + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] += to_f32(src[i]);
}

__global__ void remember_last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ token_from,
                                           const int* __restrict__ token_src, const int* __restrict__ seq_start,
                                           const int* __restrict__ seq_slot, int* __restrict__ last_token, int B,
                                           int vocab) {
  pdl_wait();   // every block of the kernel before has read `last_token`
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) last_token[seq_slot[b]] = step_token(tokens, token_from, token_src, seq_start[b + 1] - 1, vocab);
}

extern "C" int TL_NAME(tl_pair_embed_add)(const int* tokens, const int* token_from, const int* token_src,
                                          const int* token_pos, const int* token_seq, const int* seq_slot,
                                          const int* seq_start, int* last_token, const void* table, float* x,
                                          int T, int B, int H, int vocab, int buckets, long long mul_prev,
                                          long long mul_cur, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (buckets <= 0) return TL_ERR_BAD_ARG;
  const int rc = tl_launch(pair_embed_add_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, tokens,
                           token_from, token_src, token_pos, token_seq, seq_slot, seq_start,
                           (const int*)last_token, (const act_t*)table, x, H, vocab, buckets, mul_prev, mul_cur);
  if (rc != 0) return rc;
  return tl_launch(remember_last_token_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, token_from,
                   token_src, seq_start, seq_slot, last_token, B, vocab);
}

// ---------------------------------------------------------------------------
// x[r, :] += m * g * y[r, :] / sqrt(mean(y[r, :]^2) + eps); g is one number.  With `xb` given,
// xb[r, :] = the new x[r, :] in the activation type.  y: [rows, H] 32-bit, row stride ldy.
// ---------------------------------------------------------------------------
#define BRANCH_KEEP 8
__global__ void branch_norm_add_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ gain,
                                       float m, float eps, float* __restrict__ x, act_t* __restrict__ xb,
                                       int H) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float* yr = y + (size_t)r * ldy;
  float* xr = x + (size_t)r * H;
  const bool fits = H <= (int)blockDim.x * BRANCH_KEEP;
  float keep[BRANCH_KEEP];
  float ss = 0.0f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < BRANCH_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      keep[j] = i < H ? yr[i] : 0.0f;
      ss = fmaf(keep[j], keep[j], ss);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
  const float g = gain[0];
  if (fits) {
#pragma unroll
    for (int j = 0; j < BRANCH_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < H) {
        const float v = xr[i] + m * ((keep[j] / rms) * g);
        xr[i] = v;
        if (xb) xb[(size_t)r * H + i] = from_f32<act_t>(v);
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = xr[i] + m * ((yr[i] / rms) * g);
      xr[i] = v;
      if (xb) xb[(size_t)r * H + i] = from_f32<act_t>(v);
    }
  }
}

extern "C" int TL_NAME(tl_branch_norm_add)(const float* y, int ldy, const float* gain, float m, float eps,
                                           float* x, void* xb, int rows, int H, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || gain == nullptr) return TL_ERR_BAD_ARG;
  const int threads = H <= 1024 ? 128 : H <= 2048 ? 256 : 512;      // 8 values a thread up to 4096
  return tl_launch(branch_norm_add_kernel, dim3(rows), dim3(threads), 0, stream, y, ldy, gain, m, eps, x,
                   (act_t*)xb, H);
}

// ---------------------------------------------------------------------------
// out[r, :] = a N(z) + b N(z^2) + c N(z^3) + e over a row z of F numbers, powers taken element by
// element, N(u) = u / sqrt(mean(u^2) + eps); coeff = (a, b, c, e).  z 32-bit with row stride ldz.
// ---------------------------------------------------------------------------
// KEEP: values a thread keeps in registers (the row is read once if it fits KEEP * threads).
template <int POLY_KEEP>
__global__ void poly_norm_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coeff,
                                 float eps, act_t* __restrict__ out, int F) {
  __shared__ float sums[3][33];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float* zr = z + (size_t)r * ldz;
  // the row is read once and kept in registers if it fits, else read a second time
  const bool fits = F <= (int)blockDim.x * POLY_KEEP;
  float keep[POLY_KEEP];
  float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
  if (fits) {
#pragma unroll
    for (int j = 0; j < POLY_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      const float v = i < F ? zr[i] : 0.0f, v2 = v * v, v3 = v2 * v;
      keep[j] = v;
      s2 = fmaf(v, v, s2);
      s4 = fmaf(v2, v2, s4);
      s6 = fmaf(v3, v3, s6);
    }
  } else {
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
      const float v = zr[i], v2 = v * v, v3 = v2 * v;
      s2 = fmaf(v, v, s2);
      s4 = fmaf(v2, v2, s4);
      s6 = fmaf(v3, v3, s6);
    }
  }
  // the three sums in one pass through shared memory
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    s2 = warp_sum(s2); s4 = warp_sum(s4); s6 = warp_sum(s6);
    if (lane == 0) { sums[0][warp] = s2; sums[1][warp] = s4; sums[2][warp] = s6; }
    __syncthreads();
    if (warp < 3) {
      float t = lane < nwarps ? sums[warp][lane] : 0.0f;
      t = warp_sum(t);
      if (lane == 0) sums[warp][32] = t;
    }
    __syncthreads();
    s2 = sums[0][32]; s4 = sums[1][32]; s6 = sums[2][32];
  }
  const float r1 = sqrtf(s2 / (float)F + eps), r2 = sqrtf(s4 / (float)F + eps), r3 = sqrtf(s6 / (float)F + eps);
#if TL_DTYPE == 0
  // the 32-bit path divides every value, as its other norms do
#define POLY_N(v, r) ((v) / (r))
  const float a = coeff[0], b = coeff[1], c = coeff[2], e = coeff[3];
#else
  // rounded to bfloat16 afterwards: one division per row and power, folded into the coefficients
#define POLY_N(v, r) (v)
  const float a = coeff[0] / r1, b = coeff[1] / r2, c = coeff[2] / r3, e = coeff[3];
#endif
  if (fits) {
#pragma unroll
    for (int j = 0; j < POLY_KEEP; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < F) {
        const float v = keep[j], v2 = v * v, v3 = v2 * v;
        out[(size_t)r * F + i] = from_f32<act_t>(a * POLY_N(v, r1) + b * POLY_N(v2, r2) + c * POLY_N(v3, r3) + e);
      }
    }
  } else {
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
      const float v = zr[i], v2 = v * v, v3 = v2 * v;
      out[(size_t)r * F + i] = from_f32<act_t>(a * POLY_N(v, r1) + b * POLY_N(v2, r2) + c * POLY_N(v3, r3) + e);
    }
  }
}

#undef POLY_N

extern "C" int TL_NAME(tl_poly_norm)(const float* z, int ldz, const float* coeff, float eps, void* out, int rows,
                                     int F, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (F <= 0 || coeff == nullptr) return TL_ERR_BAD_ARG;
  const int threads = F <= 1024 ? 128 : F <= 4096 ? 256 : 512;
  const int per = (F + threads - 1) / threads;
  if (per <= 8)
    return tl_launch(poly_norm_kernel<8>, dim3(rows), dim3(threads), 0, stream, z, ldz, coeff, eps, (act_t*)out, F);
  if (per <= 16)
    return tl_launch(poly_norm_kernel<16>, dim3(rows), dim3(threads), 0, stream, z, ldz, coeff, eps, (act_t*)out, F);
  return tl_launch(poly_norm_kernel<32>, dim3(rows), dim3(threads), 0, stream, z, ldz, coeff, eps, (act_t*)out, F);
}
