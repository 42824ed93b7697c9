// Attention through low-rank latents over a paged cache of one vector per position.
//
// A position's cached vector is [c (rank numbers, normalised) | r (rot numbers, rotated)]: the
// compressed keys/values and the rotated key part that all heads share.  A head's key is W_uk c
// and its value W_uv c, but neither is ever formed: the query's unrotated part is carried into
// the latent space once (qa = W_uk^T q), scores are (qa . c + q_rot . r) * scale, the weighted
// sum of the c's is taken, and W_uv is applied to that sum.  Per position and head the work is
// then that of one key head of width rank + rot shared by all query heads, and the cache holds
// rank + rot numbers per position whatever the number of heads.
//
// Three kernels: what is written per token (latent_prep), products with one small matrix per
// head (headwise_gemm: qa, and the value up-projection with the output gate in its epilogue),
// and the attention itself.  Norms, angles, scores, the softmax and its sums are 32-bit.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Per token, from the 32-bit down-projections:
//   cq[t, :]  = dq[t, :] / rms * wq                          (query latent, activation type)
//   page row  = [ dkv[t, :rank] / rms * wc | rotate(dkv[t, rank:rank+rot]) ]   at the token's place
// Rotation: entry i of the rot part pairs with entry i + dims/2 (i < dims/2), angle =
// position * inv_freq[i]; entries from `dims` on pass unchanged.
// ---------------------------------------------------------------------------
__global__ void latent_prep_kernel(const float* __restrict__ dq, int ld_dq, const float* __restrict__ dkv,
                                   int ld_dkv, const float* __restrict__ wq, const float* __restrict__ wc,
                                   float eps, act_t* __restrict__ cq, act_t* __restrict__ pages,
                                   const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                                   const int* __restrict__ seq_slot, const int* __restrict__ page_table,
                                   int table_stride, const float* __restrict__ inv_freq, int q_rank, int rank,
                                   int rot, int dims) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* a = dq + (size_t)t * ld_dq;
  const float* b = dkv + (size_t)t * ld_dkv;
  float sq = 0.0f, sc = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq = fmaf(a[i], a[i], sq);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) sc = fmaf(b[i], b[i], sc);
  sq = block_sum(sq, scratch);
  sc = block_sum(sc, scratch);
  const float rq = sqrtf(sq / (float)q_rank + eps), rc = sqrtf(sc / (float)rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_f32<act_t>((a[i] / rq) * wq[i]);
  const int pos = token_pos[t];
  const int page = page_table[(size_t)seq_slot[token_seq[t]] * table_stride + pos / TL_PAGE];
  const int width = rank + rot;
  act_t* row = pages + ((size_t)page * TL_PAGE + (pos % TL_PAGE)) * width;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_f32<act_t>((b[i] / rc) * wc[i]);
  const int half = dims >> 1;
  const float* r = b + rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float u = r[i], v = r[i + half];
    row[rank + i] = from_f32<act_t>(u * cs - v * sn);
    row[rank + i + half] = from_f32<act_t>(v * cs + u * sn);
  }
  for (int i = dims + threadIdx.x; i < rot; i += blockDim.x) row[rank + i] = from_f32<act_t>(r[i]);
}

extern "C" int TL_NAME(tl_latent_prep)(const float* dq, int ld_dq, const float* dkv, int ld_dkv, const float* wq,
                                       const float* wc, float eps, void* cq, void* pages, const int* token_pos,
                                       const int* token_seq, const int* seq_slot, const int* page_table,
                                       int table_stride, const float* inv_freq, int T, int q_rank, int rank,
                                       int rot, int dims, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || rank <= 0 || rot < 0 || dims < 0 || dims > rot || (dims & 1)) return TL_ERR_BAD_ARG;
  return tl_launch(latent_prep_kernel, dim3(T), dim3(128), 0, stream, dq, ld_dq, dkv, ld_dkv, wq, wc, eps,
                   (act_t*)cq, (act_t*)pages, token_pos, token_seq, seq_slot, page_table, table_stride, inv_freq,
                   q_rank, rank, rot, dims);
}

// ---------------------------------------------------------------------------
// One small product per head:  C[t, h, n] = sum_k A[t, h, k] * W[h, n, k]
//   A 32-bit, row stride lda, head h at column h * a_head;  W [heads, N, K] in the activation type;
//   C row stride ldc, head h at column h * c_head.
// epilogue 0: C 32-bit = product;  1: C (activation type) = product * sigmoid(G[t, h * N + n]),
// G 32-bit with row stride ldg (an output gate).
// 64 x 64 tiles, 16 K-elements a step, 256 threads with 4 x 4 outputs each; 32-bit FFMA.
// ---------------------------------------------------------------------------
#define HW_BM 64
#define HW_BN 64
#define HW_BK 16

template <int EPI>
__global__ void __launch_bounds__(256)
headwise_gemm_kernel(const float* __restrict__ A, int lda, int a_head, const act_t* __restrict__ W,
                     void* __restrict__ C, int ldc, int c_head, const float* __restrict__ G, int ldg, int M,
                     int N, int K) {
  __shared__ float As[HW_BK][HW_BM + 4];
  __shared__ float Ws[HW_BK][HW_BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int h = blockIdx.z;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * HW_BM, n0 = blockIdx.x * HW_BN;
  const float* Ah = A + (size_t)h * a_head;
  const act_t* Wh = W + (size_t)h * N * K;
  float acc[4][4] = {};
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += HW_BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + j][lrow] = (am < M && k < K) ? Ah[(size_t)am * lda + k] : 0.0f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(Wh[(size_t)wn * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HW_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const size_t at = (size_t)m * ldc + (size_t)h * c_head + n;
      if (EPI == 0) {
        ((float*)C)[at] = acc[i][j];
      } else {
        const float g = G[(size_t)m * ldg + (size_t)h * N + n];
        ((act_t*)C)[at] = from_f32<act_t>(acc[i][j] * (1.0f / (1.0f + expf(-g))));
      }
    }
  }
}

// Few rows (decode): a warp per (row, head, output) streams one row of W.
template <int EPI>
__global__ void __launch_bounds__(256)
headwise_gemv_kernel(const float* __restrict__ A, int lda, int a_head, const act_t* __restrict__ W,
                     void* __restrict__ C, int ldc, int c_head, const float* __restrict__ G, int ldg, int M,
                     int N, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int h = blockIdx.z, m = blockIdx.y;
  if (n >= N) return;
  const float* a = A + (size_t)m * lda + (size_t)h * a_head;
  const act_t* w = W + ((size_t)h * N + n) * K;
  float acc = 0.0f;
  for (int k = lane; k < K; k += 32) acc = fmaf(a[k], to_f32(w[k]), acc);
  acc = warp_sum(acc);
  if (lane == 0) {
    const size_t at = (size_t)m * ldc + (size_t)h * c_head + n;
    if (EPI == 0) {
      ((float*)C)[at] = acc;
    } else {
      const float g = G[(size_t)m * ldg + (size_t)h * N + n];
      ((act_t*)C)[at] = from_f32<act_t>(acc * (1.0f / (1.0f + expf(-g))));
    }
  }
}

extern "C" int TL_NAME(tl_headwise_gemm)(const float* A, int lda, int a_head, const void* W, void* C, int ldc,
                                         int c_head, const float* G, int ldg, int M, int N, int K, int heads,
                                         int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || epilogue < 0 || epilogue > 1 || (epilogue == 1 && G == nullptr)) return TL_ERR_BAD_ARG;
  if (heads > 65535) return TL_ERR_UNSUPPORTED;
  if (M <= 16) {
    dim3 grid((N + 7) / 8, M, heads);
    if (epilogue == 0)
      return tl_launch(headwise_gemv_kernel<0>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C,
                       ldc, c_head, G, ldg, M, N, K);
    return tl_launch(headwise_gemv_kernel<1>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                     c_head, G, ldg, M, N, K);
  }
  dim3 grid((N + HW_BN - 1) / HW_BN, (M + HW_BM - 1) / HW_BM, heads);
  if (grid.y > 65535) return TL_ERR_UNSUPPORTED;
  if (epilogue == 0)
    return tl_launch(headwise_gemm_kernel<0>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                     c_head, G, ldg, M, N, K);
  return tl_launch(headwise_gemm_kernel<1>, grid, dim3(256), 0, stream, A, lda, a_head, (const act_t*)W, C, ldc,
                   c_head, G, ldg, M, N, K);
}

// ---------------------------------------------------------------------------
// The attention.  One block per (token, head): the query [qa (rank) | rotate(q_rot) (rot)] times
// `scale` lies in shared memory; keys are the page rows of positions max(0, p - W + 1) .. p (W = 0:
// from 0), taken 128 at a time from the first visible one with a running maximum and sum, so a
// position's result is the same in whatever step or batch it is computed.  The weighted sum of
// the rows' first `rank` numbers goes to o[t, h, :] (32-bit).
//   qa [T, ld_qa] 32-bit, head h's latent-space query at h * qa_head;  q [T, ldq] 32-bit, head h's
//   part to rotate at h * q_head + q_off (both may lie in one buffer)
// ---------------------------------------------------------------------------
#define LAT_THREADS 128
#define LAT_MAX_PER_THREAD 8   // rank <= 1024

#if TL_DTYPE == 0
#define LVEC 4
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
#else
#define LVEC 8
__device__ __forceinline__ void load_row_vec(const act_t* p, float* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
#endif

__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_kernel(const float* __restrict__ qa, int ld_qa, int qa_head, const float* __restrict__ q, int ldq,
                   int q_head, int q_off,
                   const act_t* __restrict__ pages, float* __restrict__ o, const int* __restrict__ token_pos,
                   const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                   const int* __restrict__ page_table, int table_stride, const float* __restrict__ inv_freq,
                   int heads, int rank, int rot, int dims, int window, float scale) {
  extern __shared__ float qs[];          // [rank + rot]
  __shared__ float ps[LAT_THREADS];
  __shared__ int pg[LAT_THREADS];
  __shared__ float scratch[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int width = rank + rot;
  const int pos = token_pos[t];
  const int* table = page_table + (size_t)seq_slot[token_seq[t]] * table_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const bool vec = width % LVEC == 0;     // rows then start on 16-byte boundaries
  for (int i = tid; i < rank; i += LAT_THREADS) qs[i] = qa[(size_t)t * ld_qa + (size_t)h * qa_head + i] * scale;
  {
    const float* r = q + (size_t)t * ldq + (size_t)h * q_head + q_off;
    const int half = dims >> 1;
    for (int i = tid; i < half; i += LAT_THREADS) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      const float u = r[i], v = r[i + half];
      qs[rank + i] = (u * cs - v * sn) * scale;
      qs[rank + i + half] = (v * cs + u * sn) * scale;
    }
    for (int i = dims + tid; i < rot; i += LAT_THREADS) qs[rank + i] = r[i] * scale;
  }
  __syncthreads();
  float m_run = -INFINITY, l_run = 0.0f;
  float acc[LAT_MAX_PER_THREAD];
#pragma unroll
  for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) acc[j] = 0.0f;
  for (int base = lo; base <= pos; base += LAT_THREADS) {
    const int i = base + tid;
    const bool valid = i <= pos;
    float s = -INFINITY;
    int page = -1;
    if (valid) {
      page = table[i / TL_PAGE];
      const act_t* krow = pages + ((size_t)page * TL_PAGE + (i % TL_PAGE)) * width;
      float dot = 0.0f;
      if (vec) {
        for (int d = 0; d < width; d += LVEC) {
          float kv[LVEC];
          load_row_vec(krow + d, kv);
#pragma unroll
          for (int e = 0; e < LVEC; ++e) dot = fmaf(qs[d + e], kv[e], dot);
        }
      } else {
        for (int d = 0; d < width; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
      }
      s = dot;
    }
    const float cmax = block_max(s, scratch);
    const float m_new = fmaxf(m_run, cmax);
    const float p = valid ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    pg[tid] = page;
    const float csum = block_sum(p, scratch);   // its barriers publish ps and pg
    const float alpha = expf(m_run - m_new);    // 0 at the first chunk
    l_run = l_run * alpha + csum;
    m_run = m_new;
    const int cnt = (pos - base + 1 < LAT_THREADS) ? pos - base + 1 : LAT_THREADS;
#pragma unroll
    for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) {
      const int d = tid + j * LAT_THREADS;
      if (d < rank) {
        float a = acc[j] * alpha;
        for (int k = 0; k < cnt; ++k) {
          const act_t* vrow = pages + ((size_t)pg[k] * TL_PAGE + ((base + k) % TL_PAGE)) * width;
          a = fmaf(ps[k], to_f32(vrow[d]), a);
        }
        acc[j] = a;
      }
    }
    __syncthreads();   // ps and pg are rewritten by the next chunk
  }
  float* orow = o + ((size_t)t * heads + h) * rank;
#pragma unroll
  for (int j = 0; j < LAT_MAX_PER_THREAD; ++j) {
    const int d = tid + j * LAT_THREADS;
    if (d < rank) orow[d] = acc[j] / l_run;
  }
}

extern "C" int TL_NAME(tl_latent_attn)(const float* qa, int ld_qa, int qa_head, const float* q, int ldq,
                                       int q_head, int q_off,
                                       const void* pages, float* o, const int* token_pos, const int* token_seq,
                                       const int* seq_slot, const int* page_table, int table_stride,
                                       const float* inv_freq, int T, int heads, int rank, int rot, int dims,
                                       int window, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || rank <= 0 || rot < 0 || dims > rot || (dims & 1)) return TL_ERR_BAD_ARG;
  if (rank > LAT_THREADS * LAT_MAX_PER_THREAD || heads > 65535 || (rank + rot) * sizeof(float) > 40 * 1024)
    return TL_ERR_UNSUPPORTED;
  return tl_launch(latent_attn_kernel, dim3(T, heads), dim3(LAT_THREADS), (size_t)(rank + rot) * sizeof(float),
                   stream, qa, ld_qa, qa_head, q, ldq, q_head, q_off, (const act_t*)pages, o, token_pos, token_seq, seq_slot,
                   page_table, table_stride, inv_freq, heads, rank, rot, dims, window, scale);
}
