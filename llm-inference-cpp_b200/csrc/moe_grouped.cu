// Routed experts for MANY tokens (a prompt): the (token, choice) items are grouped by expert and every expert's
// products run as tensor-core tiles over its own rows, so an expert's weights are read once per 64 of its items
// instead of once per item.
//
//   llmi_moe_group       one block: items per expert, their offsets, the items in expert order, where each item went,
//                        and the list of 64-row tiles (expert, first row) that the product kernels walk
//   llmi_moe_up_grouped  tile x 64 columns: a = act(h Wgᵀ) * (h Wuᵀ) for the tile's gathered token rows   -> bf16 [items, F]
//                        (experts without a gate matrix, wg null: a = act(h Wuᵀ))
//   llmi_moe_down_grouped tile x 64 columns: y = a Wdᵀ                                                     -> fp32 [items, W]
//   llmi_moe_combine     per token: sum over its choices, in the order of the choice, of weight * y[item]   -> fp32 [T, W]
// mma.sync m16n8k16 (bf16 in, fp32 accumulate), operands by cp.async through three stages of 64 k.  A row's result does not
// depend on which tile or where in a tile it lies, and the combine adds in the order of the choice: a token's output
// does not depend on its batch.  Needs W % 8 == 0 and F % 8 == 0 (16-byte rows); bf16 only.
#include <math.h>

#include "common.cuh"
#include "mma_sync.cuh"

namespace llmi {

constexpr int GB_M = 64, GB_N = 64, GB_K = 64, GB_LD = GB_K + 8, GB_STAGES = 3;
constexpr int GB_CH = GB_K / 8;            // 16-byte pieces of a tile row
constexpr int GB_SLOTS = GB_M * GB_CH / 128;   // pieces a thread copies per operand and stage

// meta: [0] number of tiles; offsets [E + 1]; tile_expert, tile_row0 [max_tiles]
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* __restrict__ idx, int n_items, int E, int32_t* __restrict__ offsets,
                 int32_t* __restrict__ sorted_items, int32_t* __restrict__ item_pos, int32_t* __restrict__ tile_expert,
                 int32_t* __restrict__ tile_row0, int32_t* __restrict__ n_tiles) {
  __shared__ int cnt[256], cursor[256];
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int e = idx[i];
    if (e >= 0) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      cursor[e] = run;
      offsets[e] = run;
      for (int r = 0; r < cnt[e]; r += GB_M) {
        tile_expert[tiles] = e;
        tile_row0[tiles] = run + r;
        ++tiles;
      }
      run += cnt[e];
    }
    offsets[E] = run;
    *n_tiles = tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int e = idx[i];
    int pos = -1;
    if (e >= 0) {
      pos = atomicAdd(&cursor[e], 1);
      sorted_items[pos] = i;
    }
    item_pos[i] = pos;
  }
}

// MODE 0: A rows are gathered token rows (item / top) of h, two weight matrices (gate, up), out = act(g) * u in bf16.
// MODE 1: A rows are the sorted rows themselves, one weight matrix, out = fp32.
// MODE 3: as MODE 0 for experts without a gate matrix: one weight matrix, out = act(h Wuᵀ) in bf16.
// MODE 2: no experts — a batch of equal products, one per head (blockIdx.z): A rows are the M rows of x from column
//         b * a_batch on, the weight is B0[b], out (bf16) goes to column b * o_batch on.
template <int MODE, int ACT>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const __nv_bfloat16* __restrict__ A, long lda, const int32_t* __restrict__ sorted_items, int top,
                   const __nv_bfloat16* __restrict__ B0, const __nv_bfloat16* __restrict__ B1, int N, int K,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ tile_expert,
                   const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ n_tiles, void* __restrict__ out, long ldo,
                   int M, long a_batch, long o_batch) {
  extern __shared__ __align__(16) unsigned char gb_smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int tile = blockIdx.x;
  if (MODE != 2 && tile >= *n_tiles) return;
  constexpr int NB = MODE == 0 ? 2 : 1;
  constexpr int STAGE = (1 + NB) * GB_M * GB_LD;              // elements per stage (GB_M == GB_N)
  __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(gb_smem);
  const int e = MODE == 2 ? (int)blockIdx.z : tile_expert[tile];
  const int row0 = MODE == 2 ? tile * GB_M : tile_row0[tile];
  const int rows_here = min(GB_M, (MODE == 2 ? M : offsets[e + 1]) - row0);
  const int n0 = blockIdx.y * GB_N;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;

  // the (row, 8-element piece) slots of a 64 x GB_K tile that this thread copies
  const __nv_bfloat16* a_src[GB_SLOTS];
  const __nv_bfloat16* b_src[NB][GB_SLOTS];
  int slot_r[GB_SLOTS], slot_c[GB_SLOTS];
#pragma unroll
  for (int i = 0; i < GB_SLOTS; ++i) {
    const int s = tid + 128 * i;
    slot_r[i] = s / GB_CH;
    slot_c[i] = (s % GB_CH) * 8;
    const int r = slot_r[i];
    if (r < rows_here) {
      const long src_row = (MODE == 0 || MODE == 3) ? (long)(sorted_items[row0 + r] / top) : (long)(row0 + r);
      a_src[i] = A + src_row * lda + (MODE == 2 ? (long)e * a_batch : 0L);
    } else {
      a_src[i] = nullptr;
    }
    const int n = n0 + r;
    b_src[0][i] = n < N ? B0 + ((size_t)e * N + n) * K : nullptr;
    if (NB == 2) b_src[1][i] = n < N ? B1 + ((size_t)e * N + n) * K : nullptr;
  }
  auto load = [&](int stage, int k0) {
    __nv_bfloat16* base = sm + (size_t)stage * STAGE;
#pragma unroll
    for (int i = 0; i < GB_SLOTS; ++i) {
      const int k = k0 + slot_c[i];
      const bool k_ok = k < K;
      __nv_bfloat16* dst = base + slot_r[i] * GB_LD + slot_c[i];
      const bool a_ok = k_ok && a_src[i] != nullptr;
      cp_async16(dst, a_ok ? (const void*)(a_src[i] + k) : (const void*)A, a_ok ? 16 : 0);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const bool b_ok = k_ok && b_src[b][i] != nullptr;
        cp_async16(dst + (1 + b) * GB_M * GB_LD, b_ok ? (const void*)(b_src[b][i] + k) : (const void*)B0, b_ok ? 16 : 0);
      }
    }
  };

  float acc[NB][2][4][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[b][mi][nt][x] = 0.f;

  const int n_k = (K + GB_K - 1) / GB_K;
#pragma unroll
  for (int s = 0; s < GB_STAGES - 1; ++s) {
    if (s < n_k) load(s, s * GB_K);
    cp_async_commit();
  }
  for (int kt = 0; kt < n_k; ++kt) {
    cp_async_wait<GB_STAGES - 2>();
    __syncthreads();                                          // stage kt is here; stage kt-1 is read out
    if (kt + GB_STAGES - 1 < n_k) load((kt + GB_STAGES - 1) % GB_STAGES, (kt + GB_STAGES - 1) * GB_K);
    cp_async_commit();
    const __nv_bfloat16* As = sm + (size_t)(kt % GB_STAGES) * STAGE;
#pragma unroll
    for (int kk = 0; kk < GB_K; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) ldsm_x4(af[mi], As + (wm * 32 + mi * 16 + (lane & 15)) * GB_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const __nv_bfloat16* Bs = As + (1 + b) * GB_M * GB_LD;
#pragma unroll
        for (int nj = 0; nj < 2; ++nj) {
          uint32_t bf[4];
          ldsm_x4(bf, Bs + (wn * 32 + nj * 16 + (lane >> 4) * 8 + (lane & 7)) * GB_LD + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma_bf16(acc[b][mi][2 * nj], af[mi], bf[0], bf[1]);
            mma_bf16(acc[b][mi][2 * nj + 1], af[mi], bf[2], bf[3]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + mi * 16 + g + 8 * half;
      if (r >= rows_here) continue;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int c = n0 + wn * 32 + nt * 8 + 2 * tq;
        if (c >= N) continue;
        const float v0 = acc[0][mi][nt][2 * half], v1 = acc[0][mi][nt][2 * half + 1];
        if (MODE == 2) {
          __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)(row0 + r) * ldo + (size_t)e * o_batch + c;
          if (c + 1 < N) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
          else dst[0] = __float2bfloat16_rn(v0);
        } else if (MODE == 3) {
          const float r0 = fmaxf(v0, 0.f), r1 = fmaxf(v1, 0.f);
          const float a0 = ACT == 2 ? r0 * r0 : ACT == 0 ? v0 / (1.0f + expf(-v0)) : 0.5f * v0 * (1.0f + tanhf(0.7978845608028654f * (v0 + 0.044715f * v0 * v0 * v0)));
          const float a1 = ACT == 2 ? r1 * r1 : ACT == 0 ? v1 / (1.0f + expf(-v1)) : 0.5f * v1 * (1.0f + tanhf(0.7978845608028654f * (v1 + 0.044715f * v1 * v1 * v1)));
          __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)(row0 + r) * ldo + c;
          if (c + 1 < N) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a0, a1);
          else dst[0] = __float2bfloat16_rn(a0);
        } else if (MODE == 0) {
          const float u0 = acc[NB - 1][mi][nt][2 * half], u1 = acc[NB - 1][mi][nt][2 * half + 1];
          const float a0 = ACT == 0 ? v0 / (1.0f + expf(-v0)) : 0.5f * v0 * (1.0f + tanhf(0.7978845608028654f * (v0 + 0.044715f * v0 * v0 * v0)));
          const float a1 = ACT == 0 ? v1 / (1.0f + expf(-v1)) : 0.5f * v1 * (1.0f + tanhf(0.7978845608028654f * (v1 + 0.044715f * v1 * v1 * v1)));
          __nv_bfloat16* dst = (__nv_bfloat16*)out + (size_t)(row0 + r) * ldo + c;
          if (c + 1 < N) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a0 * u0, a1 * u1);
          else dst[0] = __float2bfloat16_rn(a0 * u0);
        } else {
          float* dst = (float*)out + (size_t)(row0 + r) * ldo + c;
          dst[0] = v0;
          if (c + 1 < N) dst[1] = v1;
        }
      }
    }
}

// One block per token: y[t] = sum_j wt[t, j] * ys[item_pos[t * top + j]] in the order of j.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ ys, const int32_t* __restrict__ item_pos, const float* __restrict__ wt, int top,
                   int W, float* __restrict__ y, long ldy, int add) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int pos = item_pos[(size_t)t * top + j];
      if (pos >= 0) total = fmaf(wt[(size_t)t * top + j], ys[(size_t)pos * W + c], total);
    }
    y[(size_t)t * ldy + c] = add ? y[(size_t)t * ldy + c] + total : total;
  }
}

}  // namespace llmi

using namespace llmi;

// int32 entries of the grouping's scratch: offsets [E+1], sorted items and item positions [n_items] each, tile lists
// (2 x max tiles), the tile count
LLMI_EXPORT long llmi_moe_group_ints(int n_items, int E) {
  const long max_tiles = (n_items + GB_M - 1) / GB_M + E;
  return (E + 1) + 2L * n_items + 2 * max_tiles + 1;
}

LLMI_EXPORT int llmi_moe_grouped(const void* h, long ldh, const void* wg, const void* wu, const void* wd, int W, int F, int E,
                                 int top, const int32_t* idx, const float* wt, int act, int32_t* scratch, long scratch_ints,
                                 void* a_sorted, float* y_sorted, float* y, long ldy, int n_tokens, int add, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || E <= 0 || E > 256 || top <= 0) return LLMI_ERR_BAD_SIZE;
  if ((W % 8) || (F % 8) || (ldh % 8) || ((uintptr_t)h & 15) || ((uintptr_t)wg & 15) || ((uintptr_t)wu & 15) || ((uintptr_t)wd & 15) ||
      ((uintptr_t)a_sorted & 15))
    return LLMI_ERR_ALIGN;
  if (act < 0 || act > 2 || (act == 2 && wg)) return LLMI_ERR_UNSUPPORTED;
  const int n_items = n_tokens * top;
  if (scratch_ints < llmi_moe_group_ints(n_items, E)) return LLMI_ERR_BAD_SIZE;
  const int max_tiles = (n_items + GB_M - 1) / GB_M + E;
  int32_t* offsets = scratch;
  int32_t* sorted_items = offsets + (E + 1);
  int32_t* item_pos = sorted_items + n_items;
  int32_t* tile_expert = item_pos + n_items;
  int32_t* tile_row0 = tile_expert + max_tiles;
  int32_t* n_tiles = tile_row0 + max_tiles;
  int rc = launch_pdl(PDL_SMALL, moe_group_kernel, dim3(1), dim3(1024), 0, stream, idx, n_items, E, offsets, sorted_items, item_pos,
                      tile_expert, tile_row0, n_tiles);
  if (rc != LLMI_OK) return rc;
  const size_t smem_up = (size_t)GB_STAGES * 3 * GB_M * GB_LD * 2, smem_down = (size_t)GB_STAGES * 2 * GB_M * GB_LD * 2;
  const __nv_bfloat16* hb = (const __nv_bfloat16*)h;
  const __nv_bfloat16 *g = (const __nv_bfloat16*)wg, *u = (const __nv_bfloat16*)wu, *d = (const __nv_bfloat16*)wd;
  dim3 grid_up(max_tiles, (F + GB_N - 1) / GB_N), grid_down(max_tiles, (W + GB_N - 1) / GB_N);
  if (grid_up.y > 65535 || grid_down.y > 65535) return LLMI_ERR_BAD_SIZE;
  static PerDevice<bool> configured;
  if (!configured.here()) {
    cudaFuncSetAttribute(moe_grouped_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
    cudaFuncSetAttribute(moe_grouped_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
    cudaFuncSetAttribute(moe_grouped_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    cudaFuncSetAttribute(moe_grouped_kernel<3, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    cudaFuncSetAttribute(moe_grouped_kernel<3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    cudaFuncSetAttribute(moe_grouped_kernel<3, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    configured.here() = true;
  }
  if (!wg) {
#define LLMI_UNGATED(ACT)                                                                                                            \
    rc = launch_pdl(PDL_GEMM, moe_grouped_kernel<3, ACT>, grid_up, dim3(128), smem_down, stream, hb, ldh, (const int32_t*)sorted_items, \
                    top, u, u, F, W, (const int32_t*)offsets, (const int32_t*)tile_expert, (const int32_t*)tile_row0,                 \
                    (const int32_t*)n_tiles, a_sorted, (long)F, 0, 0L, 0L)
    if (act == 0) LLMI_UNGATED(0); else if (act == 1) LLMI_UNGATED(1); else LLMI_UNGATED(2);
#undef LLMI_UNGATED
  } else if (act == 0)
    rc = launch_pdl(PDL_GEMM, moe_grouped_kernel<0, 0>, grid_up, dim3(128), smem_up, stream, hb, ldh, (const int32_t*)sorted_items, top,
                    g, u, F, W, (const int32_t*)offsets, (const int32_t*)tile_expert, (const int32_t*)tile_row0,
                    (const int32_t*)n_tiles, a_sorted, (long)F, 0, 0L, 0L);
  else
    rc = launch_pdl(PDL_GEMM, moe_grouped_kernel<0, 1>, grid_up, dim3(128), smem_up, stream, hb, ldh, (const int32_t*)sorted_items, top,
                    g, u, F, W, (const int32_t*)offsets, (const int32_t*)tile_expert, (const int32_t*)tile_row0,
                    (const int32_t*)n_tiles, a_sorted, (long)F, 0, 0L, 0L);
  if (rc != LLMI_OK) return rc;
  rc = launch_pdl(PDL_GEMM, moe_grouped_kernel<1, 0>, grid_down, dim3(128), smem_down, stream, (const __nv_bfloat16*)a_sorted, (long)F,
                  (const int32_t*)sorted_items, top, d, d, W, F, (const int32_t*)offsets, (const int32_t*)tile_expert,
                  (const int32_t*)tile_row0, (const int32_t*)n_tiles, (void*)y_sorted, (long)W, 0, 0L, 0L);
  if (rc != LLMI_OK) return rc;
  return launch_pdl(PDL_SMALL, moe_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)y_sorted,
                    (const int32_t*)item_pos, wt, top, W, y, ldy, add);
}

// `batch` products of equal sizes on the tensor cores (bf16), one per head: out[:, b*by : b*by+N] = x[:, b*bx : b*bx+K] . w[b]^T,
// w [batch, N, K] contiguous.  Needs K, ldx, bx multiples of 8 and even ldo, by (16-byte operand rows, 4-byte stores).
LLMI_EXPORT int llmi_linear_heads_mma(const void* x, long ldx, long bx, const void* w, void* out, long ldo, long by, int batch, int M,
                                      int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0 || batch > 65535) return LLMI_ERR_BAD_SIZE;
  if ((K % 8) || (ldx % 8) || (bx % 8) || (ldo % 2) || (by % 2) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 3))
    return LLMI_ERR_ALIGN;
  dim3 grid((M + GB_M - 1) / GB_M, (N + GB_N - 1) / GB_N, batch);
  if (grid.y > 65535) return LLMI_ERR_BAD_SIZE;
  const size_t smem = (size_t)GB_STAGES * 2 * GB_M * GB_LD * 2;
  static PerDevice<bool> configured;
  if (!configured.here()) {
    cudaFuncSetAttribute(moe_grouped_kernel<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured.here() = true;
  }
  const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
  return launch_pdl(PDL_GEMM, moe_grouped_kernel<2, 0>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)x, ldx,
                    (const int32_t*)nullptr, 1, wb, wb, N, K, (const int32_t*)nullptr, (const int32_t*)nullptr, (const int32_t*)nullptr,
                    (const int32_t*)nullptr, out, ldo, M, bx, by);
}
