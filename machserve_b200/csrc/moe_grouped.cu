// The routed feed-forward for many rows (portions of prompts), bfloat16: the (token, expert) pairs are sorted by expert on
// the device, and each expert's rows go through its matrices in tiles on the tensor cores (mma.sync m16n8k16).
//
//   moe_sort:     counts the pairs of every expert (pairs of rows without a request are left out), lays the experts' runs
//                 side by side (offsets), writes the pairs of each run (order) and the list of tiles of 128 rows
//                 (tile_expert, tile_row0, num_tiles).  One block; nothing goes through the host, so a step that is
//                 replayed from a graph sorts its own tokens.
//   moe_grouped:  a block of four warps computes a 128 x 64 tile of one expert's product (a warp 32 rows, so that a fragment
//                 of the matrix serves two tiles of rows), K in steps of 32 through a ring of three stages of asynchronous copies.  GATED: the rows are gathered from the tokens' normed rows, two matrices
//                 (gate, up) are multiplied at once and h = act(gate) * up is written in sorted order; else the rows are
//                 the sorted h, one matrix (down), and the float32 result goes to the pair's own row.
//   moe_combine:  y[t, :] = sum_j weight[t, j] * z[t * top + j, :], j ascending, float32.
// A row's sums depend on K alone (the tile it falls into changes nothing), so a token's result does not depend on what
// else is in the batch.  K a multiple of 32.
#include "attention_mma.cuh"
#include "launch.cuh"

#define MG_BM 128
#define MG_BN 64
#define MG_BK 32
#define MG_STAGES 3
#define MG_LD (MG_BK + 8)
#define MG_MAX_EXPERTS 2048

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, const int* __restrict__ slots, int top, int experts, int pairs, int* __restrict__ offsets,
                int* __restrict__ order, int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
  __shared__ int cnt[MG_MAX_EXPERTS], cur[MG_MAX_EXPERTS];
  ms_pdl_trigger();
  ms_pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (slots[p / top] >= 0 && e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = at;
      cur[e] = at;
      for (int r = 0; r < cnt[e]; r += MG_BM) {
        tile_expert[tiles] = e;
        tile_row0[tiles] = at + r;
        ++tiles;
      }
      at += cnt[e];
    }
    offsets[experts] = at;
    *num_tiles = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (slots[p / top] >= 0 && e >= 0 && e < experts) order[atomicAdd(&cur[e], 1)] = p;
  }
}

__device__ __forceinline__ float mg_act(float g, int act) {
  if (act == 0) return g / (1.f + expf(-g));
  if (act == 2) return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));  // the exact GELU
  return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// MODE 0: the second product (rows: the sorted h; one matrix; float32 results to the pairs' own rows).  MODE 1: the first
// product of gated experts (rows gathered from the tokens; two matrices; h = act(gate) * up).  MODE 2: the first product of
// experts without a gate (rows gathered; one matrix; h = act(up)).
template <int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_kernel(const __nv_bfloat16* __restrict__ a, int lda, const int* __restrict__ order, int top,
                   const __nv_bfloat16* __restrict__ b0, const __nv_bfloat16* __restrict__ b1, int n, int k,
                   const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, const int* __restrict__ offsets,
                   const int* __restrict__ num_tiles, __nv_bfloat16* __restrict__ h, float* __restrict__ z, int act) {
  constexpr bool GATED = MODE == 1, FIRST = MODE != 0;
  constexpr int NB = GATED ? 2 : 1;
  extern __shared__ __align__(16) unsigned char mg_smem[];
  typedef __nv_bfloat16 (*ATile)[MG_BM][MG_LD];
  typedef __nv_bfloat16 (*BTile)[MG_BN][MG_LD];
  ATile a_s = reinterpret_cast<ATile>(mg_smem);                                                  // [stages][BM][LD]
  BTile b_s = reinterpret_cast<BTile>(mg_smem + sizeof(__nv_bfloat16) * MG_STAGES * MG_BM * MG_LD);  // [NB * stages][BN][LD]
  __shared__ int row_of[MG_BM];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= *num_tiles) return;
  const int e = tile_expert[tile], row0 = tile_row0[tile];
  const int rows = min(MG_BM, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * MG_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int r = tid; r < MG_BM; r += blockDim.x) row_of[r] = r < rows ? order[row0 + r] : -1;
  __syncthreads();
  // this thread's 16-byte pieces of every stage: piece tid % 4 of rows tid / 4 + 32 i (four of A's 128 rows, two of B's 64)
  const int r_a = tid >> 2, ch = tid & 3;
  const __nv_bfloat16* src_a[4];
  const __nv_bfloat16* src_b0[2];
  const __nv_bfloat16* src_b1[2];
  bool ok_a[4], ok_b[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r_a + 32 * i;
    ok_a[i] = r < rows;
    const size_t arow = ok_a[i] ? (FIRST ? (size_t)(row_of[r] / top) : (size_t)(row0 + r)) : 0;
    src_a[i] = a + arow * lda + ch * 8;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r_a + 32 * i;
    ok_b[i] = n0 + r < n;
    const size_t brow = (size_t)e * n + (ok_b[i] ? n0 + r : 0);
    src_b0[i] = b0 + brow * k + ch * 8;
    src_b1[i] = GATED ? b1 + brow * k + ch * 8 : nullptr;
  }
  auto load = [&](int stage, int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) ms_cp_async16(&a_s[stage][r_a + 32 * i][ch * 8], src_a[i] + k0, ok_a[i]);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ms_cp_async16(&b_s[stage][r_a + 32 * i][ch * 8], src_b0[i] + k0, ok_b[i]);
      if (GATED) ms_cp_async16(&b_s[MG_STAGES + stage][r_a + 32 * i][ch * 8], src_b1[i] + k0, ok_b[i]);
    }
  };
  // a warp owns 32 rows (two tiles of 16) and all 64 columns: every B fragment serves both row tiles
  float acc[NB][2][MG_BN / 8][4];
#pragma unroll
  for (int m = 0; m < NB; ++m)
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int j = 0; j < MG_BN / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][t][j][i] = 0.f;
  const int steps = k / MG_BK;
#pragma unroll
  for (int s = 0; s < MG_STAGES - 1; ++s) {
    if (s < steps) load(s, s * MG_BK);
    ms_cp_async_commit();
  }
  const int mat = lane >> 3, within = lane & 7;
  for (int kt = 0; kt < steps; ++kt) {
    ms_cp_async_wait<MG_STAGES - 2>();
    __syncthreads();  // stage kt has landed for every thread, and stage kt - 1 has been read by every warp
    if (kt + MG_STAGES - 1 < steps) load((kt + MG_STAGES - 1) % MG_STAGES, (kt + MG_STAGES - 1) * MG_BK);
    ms_cp_async_commit();
    const int st = kt % MG_STAGES;
#pragma unroll
    for (int ks = 0; ks < MG_BK / 16; ++ks) {
      unsigned af[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t)
        ms_ldmatrix_x4(af[t][0], af[t][1], af[t][2], af[t][3], &a_s[st][warp * 32 + t * 16 + within + 8 * (mat & 1)][ks * 16 + 8 * (mat >> 1)]);
#pragma unroll
      for (int m = 0; m < NB; ++m)
#pragma unroll
        for (int j = 0; j < MG_BN / 16; ++j) {
          unsigned bf[4];
          ms_ldmatrix_x4(bf[0], bf[1], bf[2], bf[3], &b_s[m * MG_STAGES + st][j * 16 + within + 8 * (mat >> 1)][ks * 16 + 8 * (mat & 1)]);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            ms_mma_bf16(acc[m][t][2 * j], af[t], bf[0], bf[1]);
            ms_mma_bf16(acc[m][t][2 * j + 1], af[t], bf[2], bf[3]);
          }
        }
    }
  }
  ms_cp_async_wait<0>();
  // rows lane / 4 and lane / 4 + 8 of each tile of 16, columns 2 * (lane % 4) and the next of every tile of 8
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = warp * 32 + t * 16 + (lane >> 2) + 8 * half;
      if (r >= rows) continue;
#pragma unroll
      for (int j = 0; j < MG_BN / 8; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + j * 8 + 2 * (lane & 3) + c;
          if (col >= n) continue;
          if (GATED)
            h[(size_t)(row0 + r) * n + col] = __float2bfloat16_rn(mg_act(acc[0][t][j][2 * half + c], act) * acc[NB - 1][t][j][2 * half + c]);
          else if (FIRST)
            h[(size_t)(row0 + r) * n + col] = __float2bfloat16_rn(mg_act(acc[0][t][j][2 * half + c], act));
          else
            z[(size_t)row_of[r] * n + col] = acc[0][t][j][2 * half + c];
        }
    }
}

static size_t mg_smem_bytes(bool gated) {
  return sizeof(__nv_bfloat16) * MG_STAGES * MG_LD * (MG_BM + (gated ? 2 : 1) * MG_BN);
}

__global__ void moe_combine_kernel(const float* __restrict__ z, const float* __restrict__ weights, const int* __restrict__ slots,
                                   float* __restrict__ y, int top, int d) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  if (slots[t] >= 0)
    for (int j = 0; j < top; ++j) s = fmaf(weights[(size_t)t * top + j], z[((size_t)t * top + j) * d + c], s);
  y[(size_t)t * d + c] = s;
}

// ints of scratch: offsets [experts + 1], order [pairs], tile_expert and tile_row0 [pairs / 128 + experts each], num_tiles [1]
MS_API long long ms_moe_grouped_scratch_ints(int pairs, int experts) {
  return (long long)(experts + 1) + pairs + 2LL * (pairs / MG_BM + experts) + 1;
}

MS_API int ms_moe_grouped_supports(int d, int ff, int experts) {
  return d > 0 && ff > 0 && d % MG_BK == 0 && ff % MG_BK == 0 && experts <= MG_MAX_EXPERTS;
}

// x [T, d] bfloat16; wg, wu [E, ff, d]; wd [E, d, ff]; ids [T, top]; weights float32 [T, top]; h [T*top, ff] bfloat16 and
// z [T*top, d] float32 scratch; y float32 [T, d].
MS_API int ms_moe_grouped(const void* x, const void* wg, const void* wu, const void* wd, const int* ids, const float* weights,
                          const int* slots, int* scratch, void* h, float* z, float* y, int tokens, int top, int d, int ff, int experts,
                          int act, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && top > 0 && act >= 0 && act <= 2, "moe_grouped: bad arguments");
  MS_REQUIRE(ms_moe_grouped_supports(d, ff, experts), "moe_grouped: sizes d=%d ff=%d experts=%d are not covered", d, ff, experts);
  const int pairs = tokens * top;
  const int max_tiles = pairs / MG_BM + experts;
  MS_REQUIRE(max_tiles <= 65535 && tokens <= 65535, "moe_grouped: %d pairs are more than one launch takes", pairs);
  int* offsets = scratch;
  int* order = offsets + experts + 1;
  int* tile_expert = order + pairs;
  int* tile_row0 = tile_expert + max_tiles;
  int* num_tiles = tile_row0 + max_tiles;
  MS_LAUNCH_RESULT("moe_sort", ms_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, 1, true, ids, slots, top, experts, pairs, offsets,
                                         order, tile_expert, tile_row0, num_tiles));
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  static bool configured = false;
  if (!configured) {
    cudaError_t e1 = cudaFuncSetAttribute(moe_grouped_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg_smem_bytes(true));
    cudaError_t e2 = cudaFuncSetAttribute(moe_grouped_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg_smem_bytes(false));
    if (e2 == cudaSuccess)
      e2 = cudaFuncSetAttribute(moe_grouped_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg_smem_bytes(false));
    MS_REQUIRE(e1 == cudaSuccess && e2 == cudaSuccess, "moe_grouped: cannot get shared memory: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    configured = true;
  }
  if (wu)
    MS_LAUNCH_RESULT("moe_grouped", ms_launch(moe_grouped_kernel<1>, dim3((ff + MG_BN - 1) / MG_BN, max_tiles), dim3(128), mg_smem_bytes(true), stream, 1, true,
                                              xb, d, (const int*)order, top, (const __nv_bfloat16*)wg, (const __nv_bfloat16*)wu, ff, d,
                                              (const int*)tile_expert, (const int*)tile_row0, (const int*)offsets, (const int*)num_tiles,
                                              (__nv_bfloat16*)h, (float*)nullptr, act));
  else  // experts without a gate: wg is their one input matrix
    MS_LAUNCH_RESULT("moe_grouped", ms_launch(moe_grouped_kernel<2>, dim3((ff + MG_BN - 1) / MG_BN, max_tiles), dim3(128), mg_smem_bytes(false), stream, 1, true,
                                              xb, d, (const int*)order, top, (const __nv_bfloat16*)wg, (const __nv_bfloat16*)nullptr, ff, d,
                                              (const int*)tile_expert, (const int*)tile_row0, (const int*)offsets, (const int*)num_tiles,
                                              (__nv_bfloat16*)h, (float*)nullptr, act));
  MS_LAUNCH_RESULT("moe_grouped", ms_launch(moe_grouped_kernel<0>, dim3((d + MG_BN - 1) / MG_BN, max_tiles), dim3(128), mg_smem_bytes(false), stream, 1, true,
                                            (const __nv_bfloat16*)h, ff, (const int*)order, top, (const __nv_bfloat16*)wd,
                                            (const __nv_bfloat16*)nullptr, d, ff, (const int*)tile_expert, (const int*)tile_row0,
                                            (const int*)offsets, (const int*)num_tiles, (__nv_bfloat16*)nullptr, z, act));
  MS_LAUNCH_RESULT("moe_combine", ms_launch(moe_combine_kernel, dim3((d + 255) / 256, tokens), dim3(256), 0, stream, 1, true, (const float*)z,
                                            weights, slots, y, top, d));
  return 0;
}
