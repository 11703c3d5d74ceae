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

#include <cuda.h>

#include "common.cuh"
#include "mma_sync.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace llmi {

constexpr int GB_M = 64, GB_N = 64, GB_K = 64, GB_LD = GB_K + 8, GB_STAGES = 3;
constexpr int GB_CH = GB_K / 8;            // 16-byte pieces of a tile row
constexpr int GB_SLOTS = GB_M * GB_CH / 128;   // pieces a thread copies per operand and stage

// meta: [0] number of tiles; offsets [E + 1]; tile_expert, tile_row0 [max_tiles]
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* __restrict__ idx, int n_items, int E, int32_t* __restrict__ offsets,
                 int32_t* __restrict__ sorted_items, int32_t* __restrict__ item_pos, int32_t* __restrict__ tile_expert,
                 int32_t* __restrict__ tile_row0, int32_t* __restrict__ n_tiles, int tile_rows) {
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
      for (int r = 0; r < cnt[e]; r += tile_rows) {
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
          const float a0 = expert_act(v0, ACT), a1 = expert_act(v1, ACT);
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
                   int W, float* __restrict__ y, long ldy, int add, const __nv_bfloat16* __restrict__ h, long ldh,
                   const float* __restrict__ id_wt) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float idw = id_wt ? id_wt[t] : 0.f;          // what the token's chosen experts that hand their input on weigh together
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int pos = item_pos[(size_t)t * top + j];
      if (pos >= 0) total = fmaf(wt[(size_t)t * top + j], ys[(size_t)pos * W + c], total);
    }
    if (idw != 0.f) total = fmaf(idw, __bfloat162float(h[(size_t)t * ldh + c]), total);
    y[(size_t)t * ldy + c] = add ? y[(size_t)t * ldy + c] + total : total;
  }
}


// ------------------------------------------------------------------------------------------------
// The grouped products of many items on the 5th-generation tensor cores (tcgen05), for experts without a gate matrix.
//
// The items' input rows are first copied into the order of the grouping (moe_gather_rows_kernel), so that a tile of
// 128 items of one expert is a box of a 2-d tensor map; the experts' weights [E, N, K] are a 3-d map whose boxes end
// at an expert's last row.  The weight tile is the 128-row operand (out features on TMEM lanes), the item tile the N
// operand (128 TMEM columns).  The grid is persistent over the units (item tile, weight-row tile), weight-row tiles
// fastest: the CTAs that run at one time share an item tile and read an expert's weights once between them.  The
// roles, the ring of stages and the two accumulators are those of the dense product (gemm_tc_kernel):
//   warp 0 : cp.async.bulk.tensor of W [128 x 64] and items [128 x 64] into a ring of stages (128-byte swizzle)
//   warp 1 : allocates TMEM; one thread issues tcgen05.mma (4 per stage) and tcgen05.commit
//   warps 2..5 : tcgen05.ld the accumulator, apply the activation, store the rows of the tile that belong to its expert
// A tile's rows past its expert's last item belong to the next expert (or to nobody): they are computed and not stored.
// Every wait on an mbarrier is bounded (an error code in *error_flag, the CTA unwinds and frees its TMEM).
constexpr int GT_BN = 128;
constexpr int GT_STAGES = 6;
constexpr int GT_A_BYTES = TC_BM * TC_BK * 2, GT_B_BYTES = GT_BN * TC_BK * 2, GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + 1024 + 8 * (2 * GT_STAGES + 4) + 16;
constexpr int GT_TMEM_COLS = 2 * GT_BN;

struct GtParams {
  int N, K;                      // an expert's weight [N, K]
  void* out;                     // [items, N], row pitch ldo: bf16 act(v) (mode 0) or fp32 v (mode 1)
  long ldo;
  int mode, act;                 // act 0: silu, 1: tanh GELU, 2: relu squared, 3: exact GELU
  const int32_t *offsets, *tile_expert, *tile_row0, *n_tiles;
  int* error_flag;
};

__device__ __forceinline__ void tma_load_3d_box(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ h, long ldh, const int32_t* __restrict__ sorted_items,
                       const int32_t* __restrict__ n_sorted, int top, int W, __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  if ((int)blockIdx.x >= *n_sorted) return;      // items of no expert (rows of no sequence) are in no group
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(sorted_items[blockIdx.x] / top) * ldh);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * W);
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void __launch_bounds__(TC_THREADS)
moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GtParams p, int m_tiles) {
  extern __shared__ uint8_t gt_smem_raw[];
  const uint32_t base = (smem_u32(gt_smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + GT_STAGES * GT_STAGE_BYTES;   // full[S], empty[S], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (GT_STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * GT_STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * GT_STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * GT_STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (p.K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    for (int s = 0; s < GT_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 4);   // the four epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)GT_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem_d;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_d) : "r"(tmem_slot));

  pdl_wait();                    // the tile lists, the item rows and the output belong to earlier kernels until now
  pdl_launch_dependents();
  const int n_units = *p.n_tiles * m_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        const int t = u / m_tiles, mt = u - t * m_tiles;
        const int e = p.tile_expert[t], row0 = p.tile_row0[t];
        for (int i = 0; i < kblocks; ++i, ++it) {
          const int s = it % GT_STAGES;
          if (it >= GT_STAGES && !mbar_wait(empty_bar(s), ((it / GT_STAGES) - 1) & 1, p.error_flag, 21)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), GT_STAGE_BYTES);
          const uint32_t a_dst = base + s * GT_STAGE_BYTES;
          tma_load_3d_box(a_dst, &map_w, i * TC_BK, mt * TC_BM, e, full_bar(s));
          tma_load_2d(a_dst + GT_A_BYTES, &map_x, i * TC_BK, row0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: D fp32, A and B bf16, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GT_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      int it = 0, j = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++j) {
        const int b = j & 1;
        if (j >= 2 && !mbar_wait(acc_empty(b), ((j >> 1) - 1) & 1, p.error_flag, 24)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_addr = tmem_d + (uint32_t)(b * GT_BN);
        for (int i = 0; i < kblocks; ++i, ++it) {
          const int s = it % GT_STAGES;
          ok = mbar_wait(full_bar(s), (it / GT_STAGES) & 1, p.error_flag, 22);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = base + s * GT_STAGE_BYTES;
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + GT_A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4)
            umma_bf16(d_addr, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(acc_full(b));
      }
    }
  } else {
    const int quad = warp & 3;   // TMEM lane quadrant
    int j = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
      const int t = u / m_tiles, mt = u - t * m_tiles;
      const int e = p.tile_expert[t], row0 = p.tile_row0[t];
      const int n_valid = min(GT_BN, p.offsets[e + 1] - row0);
      const int b = j & 1;
      const int m = mt * TC_BM + quad * 32 + lane;
      const uint32_t t_base = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * GT_BN);
      if (!mbar_wait(acc_full(b), (uint32_t)(j >> 1) & 1u, p.error_flag, 23)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c0 = 0; c0 < GT_BN; c0 += 16) {
        float v[16];
        tmem_ld16(t_base + c0, v);
        const bool last = c0 + 16 >= GT_BN || c0 + 16 >= n_valid;
        if (last) {              // the last read of this accumulator: hand it back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(b));
        }
        if (m < p.N) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (c0 + c >= n_valid) break;
            const size_t idx = (size_t)(row0 + c0 + c) * p.ldo + m;
            const float x = v[c];
            if (p.mode == 1) {
              ((float*)p.out)[idx] = x;
            } else {
              ((__nv_bfloat16*)p.out)[idx] = __float2bfloat16_rn(expert_act(x, p.act));
            }
          }
        }
        if (last) break;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)GT_TMEM_COLS));
  }
}

// A bf16 tensor map with 128-byte swizzle and boxes of [box_rows][64]: a matrix [rows, k] of row pitch ld (batch 0), or
// `batch` such matrices one after another, contiguous (boxes of one matrix: rows past its last are filled with zeros).
static int gt_make_map(CUtensorMap* map, const void* ptr, long k, long rows, long batch, long ld, int box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return LLMI_ERR_DRIVER;
    fn = (EncodeFn)sym;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)(batch ? batch : 1)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)rows * (cuuint64_t)ld * 2};
  const cuuint32_t box[3] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, batch ? 3 : 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LLMI_OK : LLMI_ERR_DRIVER;
}

}  // namespace llmi

using namespace llmi;

// int32 entries of the grouping's scratch: offsets [E+1], sorted items and item positions [n_items] each, tile lists
// (2 x max tiles), the tile count
LLMI_EXPORT long llmi_moe_group_ints(int n_items, int E) {
  const long max_tiles = (n_items + GB_M - 1) / GB_M + E;
  return (E + 1) + 2L * n_items + 2 * max_tiles + 1;
}

// id_wt (optional, fp32 [n_tokens]): a token's summed weight of chosen experts that hand their input on (choices of
// index -1): id_wt[t] * h[t] joins the token's sum in the kernel that forms it.
LLMI_EXPORT int llmi_moe_grouped(const void* h, long ldh, const void* wg, const void* wu, const void* wd, int W, int F, int E,
                                 int top, const int32_t* idx, const float* wt, int act, int32_t* scratch, long scratch_ints,
                                 void* a_sorted, float* y_sorted, float* y, long ldy, int n_tokens, int add, void* h_sorted,
                                 int* error_flag, const float* id_wt, cudaStream_t stream) {
  if (n_tokens <= 0 || W <= 0 || F <= 0 || E <= 0 || E > 256 || top <= 0) return LLMI_ERR_BAD_SIZE;
  if ((W % 8) || (F % 8) || (ldh % 8) || ((uintptr_t)h & 15) || ((uintptr_t)wg & 15) || ((uintptr_t)wu & 15) || ((uintptr_t)wd & 15) ||
      ((uintptr_t)a_sorted & 15))
    return LLMI_ERR_ALIGN;
  if (act < 0 || act > 3 || (act >= 2 && wg)) return LLMI_ERR_UNSUPPORTED;
  const int n_items = n_tokens * top;
  if (scratch_ints < llmi_moe_group_ints(n_items, E)) return LLMI_ERR_BAD_SIZE;
  // the weighted sum of a token's choices: a handful of tokens spread their columns over several blocks
  const int combine_cuts = n_tokens >= 64 ? 1 : (W + 255) / 256 < 32 ? (W + 255) / 256 : 32;
  const int max_tiles = (n_items + GB_M - 1) / GB_M + E;
  int32_t* offsets = scratch;
  int32_t* sorted_items = offsets + (E + 1);
  int32_t* item_pos = sorted_items + n_items;
  int32_t* tile_expert = item_pos + n_items;
  int32_t* tile_row0 = tile_expert + max_tiles;
  int32_t* n_tiles = tile_row0 + max_tiles;
  // Many items of experts without a gate matrix, at sizes that fill 128 x 128 tiles: the tcgen05 kernel (h_sorted lends
  // [n_items, W] bf16 for the items' input rows in the grouping's order).  LLMI_MOE_TC=0 keeps the mma.sync tiles.
  static int tc_ok = -1;
  if (tc_ok < 0) {
    const char* ev = getenv("LLMI_MOE_TC");
    tc_ok = (ev && ev[0] == '0') ? 0 : 1;
  }
  const bool tc = tc_ok && !wg && h_sorted && error_flag && n_items >= 1024 && W >= 128 && F >= 128 && !((uintptr_t)h_sorted & 15);
  int rc = launch_pdl(PDL_SMALL, moe_group_kernel, dim3(1), dim3(1024), 0, stream, idx, n_items, E, offsets, sorted_items, item_pos,
                      tile_expert, tile_row0, n_tiles, tc ? GT_BN : GB_M);
  if (rc != LLMI_OK) return rc;
  if (tc) {
    CUtensorMap mw_up, mx_up, mw_down, mx_down;
    if ((rc = gt_make_map(&mw_up, wu, W, F, E, W, TC_BM)) != LLMI_OK) return rc;
    if ((rc = gt_make_map(&mx_up, h_sorted, W, n_items, 0, W, GT_BN)) != LLMI_OK) return rc;
    if ((rc = gt_make_map(&mw_down, wd, F, W, E, F, TC_BM)) != LLMI_OK) return rc;
    if ((rc = gt_make_map(&mx_down, a_sorted, F, n_items, 0, F, GT_BN)) != LLMI_OK) return rc;
    static PerDevice<bool> tc_configured;
    if (!tc_configured.here()) {
      if (cudaFuncSetAttribute(moe_grouped_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess)
        return LLMI_ERR_LAUNCH;
      tc_configured.here() = true;
    }
    rc = launch_pdl(PDL_SMALL, moe_gather_rows_kernel, dim3(n_items), dim3(256), 0, stream, (const __nv_bfloat16*)h, ldh,
                    (const int32_t*)sorted_items, (const int32_t*)(offsets + E), top, W, (__nv_bfloat16*)h_sorted);
    if (rc != LLMI_OK) return rc;
    const int tiles_most = (n_items + GT_BN - 1) / GT_BN + E;
    const int mt_up = (F + TC_BM - 1) / TC_BM, mt_down = (W + TC_BM - 1) / TC_BM;
    GtParams pu{F, W, a_sorted, (long)F, 0, act, offsets, tile_expert, tile_row0, n_tiles, error_flag};
    GtParams pd{W, F, (void*)y_sorted, (long)W, 1, 0, offsets, tile_expert, tile_row0, n_tiles, error_flag};
    const long sms = sm_count();
    rc = launch_pdl(PDL_GEMM, moe_grouped_tc_kernel, dim3((unsigned)min((long)tiles_most * mt_up, sms)), dim3(TC_THREADS), (size_t)GT_SMEM,
                    stream, mw_up, mx_up, pu, mt_up);
    if (rc != LLMI_OK) return rc;
    rc = launch_pdl(PDL_GEMM, moe_grouped_tc_kernel, dim3((unsigned)min((long)tiles_most * mt_down, sms)), dim3(TC_THREADS),
                    (size_t)GT_SMEM, stream, mw_down, mx_down, pd, mt_down);
    if (rc != LLMI_OK) return rc;
    return launch_pdl(PDL_SMALL, moe_combine_kernel, dim3(n_tokens, combine_cuts), dim3(256), 0, stream, (const float*)y_sorted,
                      (const int32_t*)item_pos, wt, top, W, y, ldy, add, (const __nv_bfloat16*)h, ldh, id_wt);
  }
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
    cudaFuncSetAttribute(moe_grouped_kernel<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    configured.here() = true;
  }
  if (!wg) {
#define LLMI_UNGATED(ACT)                                                                                                            \
    rc = launch_pdl(PDL_GEMM, moe_grouped_kernel<3, ACT>, grid_up, dim3(128), smem_down, stream, hb, ldh, (const int32_t*)sorted_items, \
                    top, u, u, F, W, (const int32_t*)offsets, (const int32_t*)tile_expert, (const int32_t*)tile_row0,                 \
                    (const int32_t*)n_tiles, a_sorted, (long)F, 0, 0L, 0L)
    if (act == 0) LLMI_UNGATED(0); else if (act == 1) LLMI_UNGATED(1); else if (act == 2) LLMI_UNGATED(2); else LLMI_UNGATED(3);
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
  return launch_pdl(PDL_SMALL, moe_combine_kernel, dim3(n_tokens, combine_cuts), dim3(256), 0, stream, (const float*)y_sorted,
                    (const int32_t*)item_pos, wt, top, W, y, ldy, add, (const __nv_bfloat16*)h, ldh, id_wt);
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
