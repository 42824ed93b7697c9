// bfloat16 kernels of the attention with a sink, capped scores and a window that keeps the first keys
// (what it computes: sink_attention.cu), for one pair of key and value sizes per library
// (-DSA_DIM, -DSA_VDIM, multiples of 16 up to 128).
//
//   sink_attn_mma_kernel     steps of many tokens: a block takes 64 consecutive tokens of one sequence
//                            and one query head; a warp takes 16 of them and one half of every page's
//                            keys (eight warps: four groups of rows times two halves, joined at the
//                            end), so that the chain of pages a tile walks costs half as much; keys and values come page by page (64 keys) into
//                            shared memory with cp.async, two pages in flight; Q K^T and P V on the
//                            tensor cores (mma.sync m16n8k16, fragments by ldmatrix from swizzled
//                            tiles: a key page is the B operand as it lies, and so is the transposed
//                            value page); scores, cap, mask, running maximum and sum in 32-bit
//                            registers; the sink opens maximum and sum; the gate and 1/sum close.
//   sink_attn_split_kernel   steps of few tokens (decode): a block takes one token, one key/value head
//                            and a share of its pages, all query heads of the group at once (the
//                            pages are read once for the group); pages come into shared memory with
//                            cp.async, the next one while this one is worked on; the tensor-core
//                            tile's 16 rows are the group's heads, each warp takes 16 of the page's
//                            keys; partial maximum, sum and output go to a buffer,
//   sink_attn_merge_kernel   which joins the shares, counts the sink once and applies the gate.
//
// The pages a query tile needs: those of the kept first keys that lie before the window's first
// page, then the window's pages up to the tile's last position; the exact visibility is a mask
// on every score: j <= i and (i - j < window or j < keep_first).
#include "common.cuh"
#include <mma.h>

#ifndef SA_DIM
#error "SA_DIM and SA_VDIM (key and value sizes) must be given by the build"
#endif
#if TL_DTYPE != 1
#error "the tensor-core attention is built for bfloat16 only"
#endif

constexpr int DIM = SA_DIM, VDIM = SA_VDIM;
constexpr int BM = 64, BN = TL_PAGE, THREADS = 128, MMA_THREADS = 256;
static_assert(TL_PAGE == 64, "a page is one key tile of 64");
static_assert(DIM % 16 == 0 && VDIM % 16 == 0 && DIM >= 16 && VDIM >= 16 && DIM <= 128 && VDIM <= 128, "sizes");
#define LOG2E 1.4426950408889634f

typedef __nv_bfloat16 bf16;

// 16-byte chunks of a row are permuted so that the eight rows an ldmatrix reads fall into eight
// different banks groups: for rows of R elements, chunk c of row r lies at chunk c ^ f(r).
template <int R>
__device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int C = R / 8;
  if (C % 8 == 0) return chunk ^ (row & 7);
  if (C == 4) return chunk ^ ((row >> 1) & 3);
  if (C % 4 == 0) return chunk ^ (row & 3);
  if (C % 2 == 0) return chunk ^ (row & 1);
  return chunk;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// tanh through one exponential and one reciprocal: 1 - 2 / (e^(2x) + 1).  Exact limits at both ends; the
// absolute error is that of the 32-bit subtraction (1e-7), so a capped score is off by cap * 1e-7 at most.
// (The hardware's tanh.approx has a relative error of 2^-11, which near the cap is cap * 5e-4 in the score;
// the second special-function call costs the prompt kernel a tenth of its time.)
__device__ __forceinline__ float tanh_fast(float x) {
  const float e = __expf(2.0f * x);
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}

// A tile's rows of R elements, contiguous in global memory, into a swizzled shared tile.
template <int R, int ROWS, int NT = MMA_THREADS>
__device__ __forceinline__ void load_tile_async(bf16* dst, const bf16* src, int tid) {
  constexpr int C = R / 8;
  for (int i = tid; i < ROWS * C; i += NT) {
    const int row = i / C, chunk = i - row * C;
    cp_async16(dst + row * R + swz<R>(row, chunk) * 8, src + (size_t)i * 8);
  }
}

struct TilePages {
  int n_kept, first_col, n_iter;
  __device__ __forceinline__ int col(int i) const { return i < n_kept ? i : first_col + (i - n_kept); }
};
// The page-table columns that queries at positions p_first .. p_last need.
__device__ __forceinline__ TilePages tile_pages(int p_first, int p_last, int window, int keep_first) {
  TilePages t;
  const int lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  t.first_col = lo / TL_PAGE;
  t.n_kept = 0;
  if (keep_first > 0 && t.first_col > 0) {
    const int last_kept = (keep_first - 1) / TL_PAGE;
    t.n_kept = (last_kept < t.first_col - 1 ? last_kept : t.first_col - 1) + 1;
  }
  t.n_iter = t.n_kept + (p_last / TL_PAGE - t.first_col + 1);
  return t;
}

__global__ void __launch_bounds__(MMA_THREADS, 2)
sink_attn_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                     const float* __restrict__ gate, int ldg, const float* __restrict__ sink,
                     bf16* __restrict__ out, const int* __restrict__ token_pos, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_slot, const int* __restrict__ page_table, int table_stride,
                     int n_seqs, int nh, int nkv, int window, int keep_first, float scale, float cap) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);               // [BM][DIM]
  bf16* Ks = Qs + BM * DIM;                                    // [2][BN][DIM]
  bf16* Vs = Ks + 2 * BN * DIM;                                // [2][VDIM][BN]
  __shared__ int tile_info[3];
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.y, kvh = h / (nh / nkv);
  if (tid == 0) {
    // the last tiles of a sequence see the most keys: they go first, so that they do not end the kernel alone
    int tile = (int)(gridDim.x - 1 - blockIdx.x), found = -1, b = 0;
    for (; b < n_seqs; ++b) {
      const int cnt = seq_start[b + 1] - seq_start[b];
      const int tiles = (cnt + BM - 1) / BM;
      if (tile < tiles) { found = b; break; }
      tile -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = seq_start[found] + tile * BM;
      const int left = seq_start[found + 1] - tile_info[1];
      tile_info[2] = left < BM ? left : BM;
    }
  }
  __syncthreads();
  const int b = tile_info[0];
  if (b < 0) return;
  const int t0 = tile_info[1], rows = tile_info[2];
  const int p_first = token_pos[t0], p_last = p_first + rows - 1;
  const int* table = page_table + (size_t)seq_slot[b] * table_stride;
  const TilePages tp = tile_pages(p_first, p_last, window, keep_first);

  // Q tile (rows beyond the sequence's end are zero) and the first page
  {
    constexpr int C = DIM / 8;
    for (int i = tid; i < BM * C; i += MMA_THREADS) {
      const int row = i / C, chunk = i - row * C;
      bf16* dst = Qs + row * DIM + swz<DIM>(row, chunk) * 8;
      if (row < rows) cp_async16(dst, q + ((size_t)(t0 + row) * nh + h) * DIM + chunk * 8);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  auto load_page = [&](int it, int buf) {
    const int page = table[tp.col(it)];
    load_tile_async<DIM, BN>(Ks + buf * BN * DIM, k_pages + ((size_t)page * nkv + kvh) * BN * DIM, tid);
    load_tile_async<BN, VDIM>(Vs + buf * VDIM * BN, v_pages + ((size_t)page * nkv + kvh) * VDIM * BN, tid);
  };
  load_page(0, 0);
  cp_async_commit();

  const int rg = warp & 3, kh = warp >> 2;                      // group of 16 rows, half of a page's keys
  const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;            // the two rows this thread holds
  const int pos0 = r0 < rows ? p_first + r0 : -1, pos1 = r1 < rows ? p_first + r1 : -1;
  // the sink is counted once: it opens the first halves' maximum and sum
  const float sk = (sink != nullptr && kh == 0) ? sink[h] * LOG2E : -INFINITY;
  float m0 = sk, m1 = sk;
  float l0 = (sink != nullptr && kh == 0) ? 1.0f : 0.0f, l1 = l0;
  float o[VDIM / 8][4];
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
  const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;
  // what this warp's 16 rows span; a warp without rows only helps to load
  const int wrows = rows - rg * 16;
  const int wp_first = p_first + rg * 16, wp_last = wp_first + (wrows < 16 ? wrows : 16) - 1;

  for (int it = 0; it < tp.n_iter; ++it) {
    const int buf = it & 1;
    if (it + 1 < tp.n_iter) load_page(it + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* Kb = Ks + buf * BN * DIM;
    const bf16* Vb = Vs + buf * VDIM * BN;
    const int key0 = tp.col(it) * TL_PAGE;
    constexpr int HN = BN / 2;                   // keys per half
    const int half = kh;
    const int kbeg = key0 + half * HN, kend = kbeg + HN - 1;     // this warp's keys of the page
    // keys that none of the warp's rows sees (after its last row, or before its first row's window and
    // not kept) are passed over; keys that all of them see need no mask
    const bool none = wrows <= 0 || kbeg > wp_last ||
                      (window > 0 && wp_first - kend >= window && kbeg >= keep_first);
    if (none) { __syncthreads(); continue; }
    const bool whole = wrows >= 16 && kend <= wp_first &&
                       (window <= 0 || wp_last - kbeg < window || kend < keep_first);
    {
      // S = Q K^T : 16 rows x 32 keys per warp
      float s[HN / 8][4];
#pragma unroll
      for (int n = 0; n < HN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < DIM / 16; ++kk) {
        unsigned qa[4];
        {
          const int row = rg * 16 + (lane & 15), chunk = kk * 2 + (lane >> 4);
          ldmatrix_x4(qa, Qs + row * DIM + swz<DIM>(row, chunk) * 8);
        }
#pragma unroll
        for (int np = 0; np < HN / 16; ++np) {
          unsigned bfr[4];
          const int row = half * HN + np * 16 + (lane >> 4) * 8 + (lane & 7), chunk = kk * 2 + ((lane >> 3) & 1);
          ldmatrix_x4(bfr, Kb + row * DIM + swz<DIM>(row, chunk) * 8);
          mma_bf16(s[2 * np], qa, bfr[0], bfr[1]);
          mma_bf16(s[2 * np + 1], qa, bfr[2], bfr[3]);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < HN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + half * HN + n * 8 + (lane & 3) * 2 + (e & 1);
          const int i = e < 2 ? pos0 : pos1;
          float v = cap > 0.0f ? cap2 * tanh_fast(s[n][e] * scale * inv_cap) : s[n][e] * scale2;
          const bool vis = whole || (j <= i && (window <= 0 || i - j < window || j < keep_first));
          v = vis ? v : -INFINITY;
          s[n][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      // (a row that has seen nothing yet and has no sink keeps -inf: its factors are taken as zero)
      const float a0 = n0 == -INFINITY ? 0.0f : exp2f(m0 - n0), a1 = n1 == -INFINITY ? 0.0f : exp2f(m1 - n1);
      const float b0 = n0 == -INFINITY ? 0.0f : n0, b1 = n1 == -INFINITY ? 0.0f : n1;
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int n = 0; n < HN / 8; ++n) {
        s[n][0] = exp2f(s[n][0] - b0); s[n][1] = exp2f(s[n][1] - b0);
        s[n][2] = exp2f(s[n][2] - b1); s[n][3] = exp2f(s[n][3] - b1);
        sum0 += s[n][0] + s[n][1];
        sum1 += s[n][2] + s[n][3];
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * a0 + sum0; l1 = l1 * a1 + sum1;
      m0 = n0; m1 = n1;
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
      // O += P V : P from the score registers, V^T rows are the B operand
#pragma unroll
      for (int kk = 0; kk < HN / 16; ++kk) {
        unsigned pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < VDIM / 16; ++np) {
          unsigned bfr[4];
          const int row = np * 16 + (lane >> 4) * 8 + (lane & 7), chunk = (half * (HN / 16) + kk) * 2 + ((lane >> 3) & 1);
          ldmatrix_x4(bfr, Vb + row * BN + swz<BN>(row, chunk) * 8);
          mma_bf16(o[2 * np], pa, bfr[0], bfr[1]);
          mma_bf16(o[2 * np + 1], pa, bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();   // the buffer is refilled two iterations on
  }
  pdl_launch_dependents();   // only now: a grid let go earlier would sit on the SMs and take issue slots
  cp_async_wait<0>();
  __syncthreads();
  // the second halves hand their sums to the first through the page buffers: [BM][VDIM] floats
  float* Om = reinterpret_cast<float*>(smem_raw);
  __shared__ float pm[BM], pl[BM];
  if (kh == 1) {
    const int a = rg * 16 + (lane >> 2), b2 = a + 8;
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n) {
      const int c = n * 8 + (lane & 3) * 2;
      Om[a * VDIM + c] = o[n][0]; Om[a * VDIM + c + 1] = o[n][1];
      Om[b2 * VDIM + c] = o[n][2]; Om[b2 * VDIM + c + 1] = o[n][3];
    }
    if ((lane & 3) == 0) { pm[a] = m0; pl[a] = l0; pm[b2] = m1; pl[b2] = l1; }
  }
  __syncthreads();
  if (kh == 1) return;
  {
    const float ma = pm[r0], mb = pm[r1];
    const float M0 = fmaxf(m0, ma), M1 = fmaxf(m1, mb);
    const float fa0 = m0 == -INFINITY ? 0.0f : exp2f(m0 - M0), fb0 = ma == -INFINITY ? 0.0f : exp2f(ma - M0);
    const float fa1 = m1 == -INFINITY ? 0.0f : exp2f(m1 - M1), fb1 = mb == -INFINITY ? 0.0f : exp2f(mb - M1);
    l0 = l0 * fa0 + pl[r0] * fb0;
    l1 = l1 * fa1 + pl[r1] * fb1;
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n) {
      const int c = n * 8 + (lane & 3) * 2;
      o[n][0] = o[n][0] * fa0 + Om[r0 * VDIM + c] * fb0;
      o[n][1] = o[n][1] * fa0 + Om[r0 * VDIM + c + 1] * fb0;
      o[n][2] = o[n][2] * fa1 + Om[r1 * VDIM + c] * fb1;
      o[n][3] = o[n][3] * fa1 + Om[r1 * VDIM + c + 1] * fb1;
    }
  }
  float f0 = 0.0f, f1 = 0.0f;
  if (r0 < rows) f0 = (gate != nullptr ? 1.0f / (1.0f + __expf(-gate[(size_t)(t0 + r0) * ldg + h])) : 1.0f) / l0;
  if (r1 < rows) f1 = (gate != nullptr ? 1.0f / (1.0f + __expf(-gate[(size_t)(t0 + r1) * ldg + h])) : 1.0f) / l1;
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) {
    const int c = n * 8 + (lane & 3) * 2;
    if (r0 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + r0) * nh + h) * VDIM + c) = pack_bf16(o[n][0] * f0, o[n][1] * f0);
    if (r1 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(t0 + r1) * nh + h) * VDIM + c) = pack_bf16(o[n][2] * f1, o[n][3] * f1);
  }
}

extern "C" int tl_sink_attn_mma(const void* q, const void* k_pages, const void* v_pages, const float* gate, int ldg,
                                const float* sink, void* out, const int* token_pos, const int* seq_start,
                                const int* seq_slot, const int* page_table, int table_stride, int T, int n_seqs,
                                int nh, int nkv, int window, int keep_first, float scale, float cap,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh > 65535) return TL_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(BM * DIM + 2 * BN * DIM + 2 * VDIM * BN) * sizeof(bf16);
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(sink_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return TL_ERR_UNSUPPORTED;
    set = true;
  }
  const int tiles = (T + BM - 1) / BM + n_seqs;      // an upper bound; a block without a tile leaves
  return tl_launch(sink_attn_mma_kernel, dim3(tiles, nh), dim3(MMA_THREADS), smem, stream, (const bf16*)q,
                   (const bf16*)k_pages, (const bf16*)v_pages, gate, ldg, sink, (bf16*)out, token_pos, seq_start,
                   seq_slot, page_table, table_stride, n_seqs, nh, nkv, window, keep_first, scale, cap);
}

// ---------------------------------------------------------------------------------------------------
// Steps of few tokens.  part: [T][nkv][splits][group][VDIM + 2] floats: output sums, then maximum (log2
// units) and sum of the share; a share without visible keys leaves maximum -inf and sum 0.
// ---------------------------------------------------------------------------------------------------
#define SPLIT_MAX_GROUP 16

// The 16 rows of the tensor-core tile are the query heads of one key/value head's group (rows beyond the
// group are zero); each of the four warps takes 16 of a page's 64 keys, with its own running maximum and
// sum, and the four are joined in shared memory at the end.
__global__ void __launch_bounds__(THREADS)
sink_attn_split_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                       float* __restrict__ part, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                       const int* __restrict__ seq_slot, const int* __restrict__ page_table, int table_stride, int nh,
                       int nkv, int window, int keep_first, float scale, float cap, int splits) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);                // [2][BN][DIM]
  bf16* Vs = Ks + 2 * BN * DIM;                                 // [2][VDIM][BN]
  __shared__ __align__(16) bf16 Qs[16 * DIM];
  __shared__ float wm[4][16], wl[4][16];
  pdl_wait();
  const int t = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = nh / nkv;
  const int pos = token_pos[t];
  const int* table = page_table + (size_t)seq_slot[token_seq[t]] * table_stride;
  const TilePages tp = tile_pages(pos, pos, window, keep_first);
  const int per = (tp.n_iter + splits - 1) / splits;
  const int i0 = sp * per, i1 = (i0 + per < tp.n_iter) ? i0 + per : tp.n_iter;
  auto load_page = [&](int it, int buf) {
    const int page = table[tp.col(it)];
    load_tile_async<DIM, BN, THREADS>(Ks + buf * BN * DIM, k_pages + ((size_t)page * nkv + kvh) * BN * DIM, tid);
    load_tile_async<BN, VDIM, THREADS>(Vs + buf * VDIM * BN, v_pages + ((size_t)page * nkv + kvh) * VDIM * BN, tid);
  };
  if (i0 < i1) load_page(i0, 0);
  cp_async_commit();
  {
    constexpr int C = DIM / 8;
    for (int i = tid; i < 16 * C; i += THREADS) {
      const int row = i / C, chunk = i - row * C;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < group) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * nh + kvh * group + row) * DIM + chunk * 8);
      *reinterpret_cast<uint4*>(Qs + row * DIM + swz<DIM>(row, chunk) * 8) = v;
    }
  }
  __syncthreads();
  unsigned qf[DIM / 16][4];
#pragma unroll
  for (int kk = 0; kk < DIM / 16; ++kk) {
    const int row = lane & 15, chunk = kk * 2 + (lane >> 4);
    ldmatrix_x4(qf[kk], Qs + row * DIM + swz<DIM>(row, chunk) * 8);
  }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  float o[VDIM / 8][4];
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
  const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;
  for (int it = i0; it < i1; ++it) {
    const int buf = (it - i0) & 1;
    if (it + 1 < i1) load_page(it + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* Kb = Ks + buf * BN * DIM;
    const bf16* Vb = Vs + buf * VDIM * BN;
    const int key0 = tp.col(it) * TL_PAGE + warp * 16;
    float s[2][4];
    s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < DIM / 16; ++kk) {
      unsigned bfr[4];
      const int row = warp * 16 + (lane >> 4) * 8 + (lane & 7), chunk = kk * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(bfr, Kb + row * DIM + swz<DIM>(row, chunk) * 8);
      mma_bf16(s[0], qf[kk], bfr[0], bfr[1]);
      mma_bf16(s[1], qf[kk], bfr[2], bfr[3]);
    }
    float mx = -INFINITY;        // every row sees the same keys: one mask, but a maximum per row
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = key0 + n * 8 + (lane & 3) * 2 + (e & 1);
        float v = cap > 0.0f ? cap2 * tanh_fast(s[n][e] * scale * inv_cap) : s[n][e] * scale2;
        const bool vis = j <= pos && (window <= 0 || pos - j < window || j < keep_first);
        v = vis ? v : -INFINITY;
        s[n][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    (void)mx;
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float a0 = n0 == -INFINITY ? 0.0f : exp2f(m0 - n0), a1 = n1 == -INFINITY ? 0.0f : exp2f(m1 - n1);
    const float b0 = n0 == -INFINITY ? 0.0f : n0, b1 = n1 == -INFINITY ? 0.0f : n1;
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      s[n][0] = exp2f(s[n][0] - b0); s[n][1] = exp2f(s[n][1] - b0);
      s[n][2] = exp2f(s[n][2] - b1); s[n][3] = exp2f(s[n][3] - b1);
      sum0 += s[n][0] + s[n][1];
      sum1 += s[n][2] + s[n][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * a0 + sum0; l1 = l1 * a1 + sum1;
    m0 = n0; m1 = n1;
    unsigned pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = pack_bf16(s[0][2], s[0][3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int np = 0; np < VDIM / 16; ++np) {
      o[2 * np][0] *= a0; o[2 * np][1] *= a0; o[2 * np][2] *= a1; o[2 * np][3] *= a1;
      o[2 * np + 1][0] *= a0; o[2 * np + 1][1] *= a0; o[2 * np + 1][2] *= a1; o[2 * np + 1][3] *= a1;
      unsigned bfr[4];
      const int row = np * 16 + (lane >> 4) * 8 + (lane & 7), chunk = warp * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(bfr, Vb + row * BN + swz<BN>(row, chunk) * 8);
      mma_bf16(o[2 * np], pa, bfr[0], bfr[1]);
      mma_bf16(o[2 * np + 1], pa, bfr[2], bfr[3]);
    }
    __syncthreads();   // this page's buffer is refilled two rounds on
  }
  pdl_launch_dependents();   // only now: a grid let go earlier would sit on the SMs and take issue slots
  cp_async_wait<0>();
  __syncthreads();
  // join the four warps' shares of the keys: [warp][row][VDIM] sums over the page buffers
  float* Om = reinterpret_cast<float*>(smem_raw);
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n) {
      const int c = n * 8 + (lane & 3) * 2;
      Om[(warp * 16 + r0) * VDIM + c] = o[n][0];
      Om[(warp * 16 + r0) * VDIM + c + 1] = o[n][1];
      Om[(warp * 16 + r1) * VDIM + c] = o[n][2];
      Om[(warp * 16 + r1) * VDIM + c + 1] = o[n][3];
    }
    if ((lane & 3) == 0) {
      wm[warp][r0] = m0; wl[warp][r0] = l0;
      wm[warp][r1] = m1; wl[warp][r1] = l1;
    }
  }
  __syncthreads();
  float* dst = part + ((((size_t)t * nkv + kvh) * splits + sp) * group) * (VDIM + 2);
  for (int g = 0; g < group; ++g) {
    const float M = fmaxf(fmaxf(wm[0][g], wm[1][g]), fmaxf(wm[2][g], wm[3][g]));
    float f[4], l = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      f[w] = wm[w][g] == -INFINITY ? 0.0f : exp2f(wm[w][g] - M);
      l += wl[w][g] * f[w];
    }
    for (int c = tid; c < VDIM; c += THREADS) {
      float a = 0.0f;
#pragma unroll
      for (int w = 0; w < 4; ++w) a += Om[(w * 16 + g) * VDIM + c] * f[w];
      dst[(size_t)g * (VDIM + 2) + c] = a;
    }
    if (tid == 0) {
      dst[(size_t)g * (VDIM + 2) + VDIM] = M;
      dst[(size_t)g * (VDIM + 2) + VDIM + 1] = l;
    }
  }
}

__global__ void __launch_bounds__(THREADS)
sink_attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ gate, int ldg,
                       const float* __restrict__ sink, bf16* __restrict__ out, int nh, int nkv, int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int group = nh / nkv, kvh = h / group, g = h - kvh * group;
  const float* src = part + (((size_t)t * nkv + kvh) * splits * group + g) * (VDIM + 2);
  const size_t stride = (size_t)group * (VDIM + 2);
  float m = sink != nullptr ? sink[h] * LOG2E : -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, src[s * stride + VDIM]);
  float l = sink != nullptr ? exp2f(sink[h] * LOG2E - m) : 0.0f;
  float a = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const float ms = src[s * stride + VDIM];
    const float w = ms == -INFINITY ? 0.0f : exp2f(ms - m);
    l += src[s * stride + VDIM + 1] * w;
    if (tid < VDIM) a += src[s * stride + tid] * w;
  }
  const float gv = gate != nullptr ? 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + h])) : 1.0f;
  if (tid < VDIM) out[((size_t)t * nh + h) * VDIM + tid] = __float2bfloat16_rn(a * gv / l);
}

extern "C" long long tl_sink_attn_split_floats(int T, int nh, int nkv, int splits) {
  return (long long)T * nkv * splits * (nh / nkv) * (VDIM + 2);
}

extern "C" int tl_sink_attn_split(const void* q, const void* k_pages, const void* v_pages, const float* gate, int ldg,
                                  const float* sink, void* out, float* part, const int* token_pos,
                                  const int* token_seq, const int* seq_slot, const int* page_table,
                                  int table_stride, int T, int nh, int nkv, int window, int keep_first, float scale,
                                  float cap, int splits, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || nh / nkv > SPLIT_MAX_GROUP || nh > 65535 || nkv > 65535 || splits < 1 ||
      splits > 65535 || part == nullptr)
    return TL_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(2 * BN * DIM + 2 * VDIM * BN) * sizeof(bf16);
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(sink_attn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return TL_ERR_UNSUPPORTED;
    set = true;
  }
  const int rc = tl_launch(sink_attn_split_kernel, dim3(T, nkv, splits), dim3(THREADS), smem, stream, (const bf16*)q,
                           (const bf16*)k_pages, (const bf16*)v_pages, part, token_pos, token_seq, seq_slot,
                           page_table, table_stride, nh, nkv, window, keep_first, scale, cap, splits);
  if (rc != 0) return rc;
  return tl_launch(sink_attn_merge_kernel, dim3(T, nh), dim3(THREADS), 0, stream, (const float*)part, gate, ldg,
                   sink, (bf16*)out, nh, nkv, splits);
}
