// Gated linear attention: a recurrent mixer with a matrix state per head and a decay per key channel.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dk, dv] per head, float32, one per request slot
//   o_t = S_t^T (q_t * q_scale)
//   a_t = sigmoid(z_t)^(1/tau) = exp(logsigmoid(z_t) / tau),  z_t = W2 u_t + b2 (u_t the low-rank projection of the token)
//   y_t = o_t / rms(o_t) * w (per head, over dv, eps inside the root) * silu(gate_t)
// Everything here is float32: the decays and their logarithms, the state, the sums, the norm and the gate.
//
// gla_decay:   a[t, n] = exp(logsigmoid(sum_r W2[n, r] * u[t, r] + b2[n]) / tau); one thread an output.
// gla_scan:    a block owns 32 (or 8) value columns of one head of one sequence and goes through the sequence's rows of the step in
//              order, from the state the step found to the state it leaves.  Thread (c, g) holds KPT consecutive key rows of
//              column c in registers; q, k and exp(g) of TB tokens at a time are staged in shared memory, the next batch on
//              its way while this one is worked on; the partial outputs of the sixteen row groups are summed in group order.
//              The arithmetic of a token depends on the tokens before it alone, not on how the sequence was cut into steps
//              or on what else is in the batch.
// gla_output:  the norm over a head's dv outputs, its weight, and the gate; one warp a (token, head).
#include "launch.cuh"

#define GLA_GROUPS 16
#define GLA_TB 16

template <typename TW>
__global__ void gla_decay_kernel(const float* __restrict__ u, int ldu, const TW* __restrict__ w2, const float* __restrict__ b2, int rank,
                                 float inv_tau, float* __restrict__ g, int n, size_t total) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / n;
  const int c = (int)(i - t * n);
  const float* ur = u + t * ldu;
  const TW* wr = w2 + (size_t)c * rank;
  float z = 0.f;
  for (int r = 0; r < rank; ++r) z = fmaf(ms_to_float(wr[r]), ur[r], z);
  z += b2 ? b2[c] : 0.f;
  // logsigmoid(z) = min(z, 0) - log1p(exp(-|z|)); the decay is the exponential of its 1/tau-th
  g[i] = expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

MS_API int ms_gla_decay(const float* u, int ldu, const void* w2, int w_dtype, const float* b2, int rank, float tau, float* g, int tokens,
                        int n, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && n > 0 && rank > 0 && ldu >= rank && tau > 0.f, "gla_decay: bad arguments tokens=%d n=%d rank=%d tau=%g", tokens, n,
             rank, tau);
  const size_t total = (size_t)tokens * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (w_dtype == MS_F32)
    MS_LAUNCH_RESULT("gla_decay", ms_launch(gla_decay_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true, u, ldu, (const float*)w2, b2,
                                            rank, 1.f / tau, g, n, total));
  else if (w_dtype == MS_BF16)
    MS_LAUNCH_RESULT("gla_decay", ms_launch(gla_decay_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true, u, ldu,
                                            (const __nv_bfloat16*)w2, b2, rank, 1.f / tau, g, n, total));
  else
    MS_REQUIRE(false, "gla_decay: unknown weight dtype %d", w_dtype);
  return 0;
}

// q, k, v: float32 rows of one product, row stride ld, at column offsets q_off, k_off, v_off; within each, head h begins at
// h*dk (q, k) or h*dv (v).  g: float32 [T, heads*dk].  state: float32 [slots, heads, dk, dv].  o: float32 [T, heads*dv].
// g holds the decays a themselves.  The rows of GLA_TB tokens at a time come into shared memory by asynchronous copies, one
// batch ahead of the one that is worked on (two places); q_scale multiplies the finished sums.
__device__ __forceinline__ void gla_cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void gla_cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

template <int KPT, int COLS>
__global__ void __launch_bounds__(COLS * GLA_GROUPS)
gla_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ g, float q_scale,
                float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
                const int* __restrict__ slot_of_token, float* __restrict__ o, int heads, int dk, int dv, int vec) {
  constexpr int KP = KPT * GLA_GROUPS;             // key rows, padded
  constexpr int ROW = 3 * KP + COLS;           // floats of one token in a stage: q | k | a | v
  extern __shared__ __align__(16) float gla_smem[];
  float* stage0 = gla_smem;                        // [2][GLA_TB][ROW]
  float* part = gla_smem + 2 * GLA_TB * ROW;       // [GLA_TB][GLA_GROUPS][COLS]
  ms_pdl_trigger();
  ms_pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int row0 = cu_tokens[seq], rows = cu_tokens[seq + 1] - row0;
  if (rows <= 0 || slot_of_token[row0] < 0) return;  // a sequence of no rows, or rows of no request
  const int slot = state_slots[seq];
  const int c = threadIdx.x % COLS, grp = threadIdx.x / COLS;
  const int col = c0 + c;
  const bool live = col < dv;
  // padding of the key rows: q = k = 0 and a = 1 for good, in both stages
  for (int e = threadIdx.x; e < 2 * GLA_TB * (KP - dk); e += blockDim.x) {
    const int tb = e / (KP - dk), r = dk + e % (KP - dk);
    float* t = stage0 + (size_t)tb * ROW;
    t[r] = 0.f;
    t[KP + r] = 0.f;
    t[2 * KP + r] = 1.f;
  }
  // one warp a token: no division in the loop; 16-byte copies where the rows allow it
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  auto request = [&](int t0, int st) {
    const int nt = min(GLA_TB, rows - t0);
    float* base = stage0 + (size_t)st * GLA_TB * ROW;
    for (int tb = warp; tb < nt; tb += nwarps) {
      const size_t t = (size_t)(row0 + t0 + tb);
      float* dst = base + (size_t)tb * ROW;
      const float* qs = proj + t * ld + q_off + h * dk;
      const float* ks = proj + t * ld + k_off + h * dk;
      const float* as = g + t * ((size_t)heads * dk) + h * dk;
      const float* vs = proj + t * ld + v_off + h * dv + c0;
      if (vec) {
        for (int r = lane * 4; r < dk; r += 128) {
          gla_cp_async16(dst + r, qs + r);
          gla_cp_async16(dst + KP + r, ks + r);
          gla_cp_async16(dst + 2 * KP + r, as + r);
        }
        for (int cc = lane * 4; cc < COLS; cc += 128) {
          if (c0 + cc < dv) gla_cp_async16(dst + 3 * KP + cc, vs + cc);  // (dv is a multiple of 4 here)
          else *reinterpret_cast<float4*>(dst + 3 * KP + cc) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
        for (int r = lane; r < dk; r += 32) {
          gla_cp_async4(dst + r, qs + r);
          gla_cp_async4(dst + KP + r, ks + r);
          gla_cp_async4(dst + 2 * KP + r, as + r);
        }
        for (int cc = lane; cc < COLS; cc += 32) {
          if (c0 + cc < dv) gla_cp_async4(dst + 3 * KP + cc, vs + cc);
          else dst[3 * KP + cc] = 0.f;
        }
      }
    }
  };
  request(0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  float* st = state + (((size_t)slot * heads + h) * dk) * dv;
  float s[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = grp * KPT + i;
    s[i] = (live && r < dk) ? st[(size_t)r * dv + col] : 0.f;
  }
  int stg = 0;
  for (int t0 = 0; t0 < rows; t0 += GLA_TB, stg ^= 1) {
    const int nt = min(GLA_TB, rows - t0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // the batch has landed for every thread; the batch before has been read and its partial sums added up
    if (t0 + GLA_TB < rows) request(t0 + GLA_TB, stg ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    float* base = stage0 + (size_t)stg * GLA_TB * ROW;
    auto token = [&](int tb) {
      const float* t = base + (size_t)tb * ROW;
      const float v = t[3 * KP + c];
      float acc0 = 0.f, acc1 = 0.f;  // two chains of sums (even and odd rows), added at the end: the order is fixed
      if constexpr (KPT % 4 == 0) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
          const float4 q = *reinterpret_cast<const float4*>(t + grp * KPT + i);
          const float4 k = *reinterpret_cast<const float4*>(t + KP + grp * KPT + i);
          const float4 a = *reinterpret_cast<const float4*>(t + 2 * KP + grp * KPT + i);
          s[i] = fmaf(a.x, s[i], k.x * v);
          s[i + 1] = fmaf(a.y, s[i + 1], k.y * v);
          s[i + 2] = fmaf(a.z, s[i + 2], k.z * v);
          s[i + 3] = fmaf(a.w, s[i + 3], k.w * v);
          acc0 = fmaf(s[i], q.x, acc0);
          acc1 = fmaf(s[i + 1], q.y, acc1);
          acc0 = fmaf(s[i + 2], q.z, acc0);
          acc1 = fmaf(s[i + 3], q.w, acc1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < KPT; i += 2) {  // (KPT is even)
          const float2 q = *reinterpret_cast<const float2*>(t + grp * KPT + i);
          const float2 k = *reinterpret_cast<const float2*>(t + KP + grp * KPT + i);
          const float2 a = *reinterpret_cast<const float2*>(t + 2 * KP + grp * KPT + i);
          s[i] = fmaf(a.x, s[i], k.x * v);
          s[i + 1] = fmaf(a.y, s[i + 1], k.y * v);
          acc0 = fmaf(s[i], q.x, acc0);
          acc1 = fmaf(s[i + 1], q.y, acc1);
        }
      }
      part[((size_t)tb * GLA_GROUPS + grp) * COLS + c] = acc0 + acc1;
    };
    if (nt == GLA_TB) {  // a full batch: unrolled, so that the loads of later tokens are on their way under the sums of earlier ones
#pragma unroll
      for (int tb = 0; tb < GLA_TB; ++tb) token(tb);
    } else {
      for (int tb = 0; tb < nt; ++tb) token(tb);
    }
    __syncthreads();
    for (int tb = grp; tb < nt; tb += GLA_GROUPS) {
      float sum = 0.f;
#pragma unroll
      for (int gi = 0; gi < GLA_GROUPS; ++gi) sum += part[((size_t)tb * GLA_GROUPS + gi) * COLS + c];
      if (live) o[(size_t)(row0 + t0 + tb) * ((size_t)heads * dv) + h * dv + col] = sum * q_scale;
    }
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = grp * KPT + i;
    if (live && r < dk) st[(size_t)r * dv + col] = s[i];
  }
}

template <int KPT, int COLS>
static int gla_scan_launch(cudaStream_t stream, int seqs, const float* proj, int ld, int q_off, int k_off, int v_off,
                           const float* g, float q_scale, float* state, const int* cu_tokens, const int* state_slots,
                           const int* slot_of_token, float* o, int heads, int dk, int dv) {
  const int vec = dk % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                  ((uintptr_t)proj | (uintptr_t)g) % 16 == 0;
  constexpr int KP = KPT * GLA_GROUPS;
  const size_t smem = (size_t)(2 * GLA_TB * (3 * KP + COLS) + GLA_TB * GLA_GROUPS * COLS) * sizeof(float);
  const dim3 grid((dv + COLS - 1) / COLS, heads, seqs), block(COLS * GLA_GROUPS);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<KPT, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "gla_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  MS_LAUNCH_RESULT("gla_scan", ms_launch(gla_scan_kernel<KPT, COLS>, grid, block, smem, stream, 1, true, proj, ld, q_off, k_off, v_off, g, q_scale,
                                         state, cu_tokens, state_slots, slot_of_token, o, heads, dk, dv, vec));
  return 0;
}

MS_API int ms_gla_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* g, float q_scale, float* state,
                       const int* cu_tokens, const int* state_slots, const int* slot_of_token, float* o, int seqs, int heads, int dk, int dv,
                       int narrow, cudaStream_t stream) {
  if (seqs == 0) return 0;
  MS_REQUIRE(seqs > 0 && heads > 0 && dk > 0 && dv > 0, "gla_scan: bad sizes seqs=%d heads=%d dk=%d dv=%d", seqs, heads, dk, dv);
  MS_REQUIRE(dk <= 16 * GLA_GROUPS, "gla_scan: %d key channels a head are more than the kernel covers (%d)", dk, 16 * GLA_GROUPS);
  MS_REQUIRE(seqs <= 65535 && heads <= 65535, "gla_scan: too many sequences or heads for one launch");
  const int kpt = (dk + GLA_GROUPS - 1) / GLA_GROUPS;
  // narrow: 8 value columns a block instead of 32, for steps whose few sequences bring many rows each (the blocks of a
  // sequence are the only parallelism a scan has); a column's arithmetic is the same either way
#define MS_GLA_GO(K)                                                                                                                     \
  return narrow ? gla_scan_launch<K, 8>(stream, seqs, proj, ld, q_off, k_off, v_off, g, q_scale, state, cu_tokens, state_slots,          \
                                        slot_of_token, o, heads, dk, dv)                                                                 \
                : gla_scan_launch<K, 32>(stream, seqs, proj, ld, q_off, k_off, v_off, g, q_scale, state, cu_tokens, state_slots,         \
                                         slot_of_token, o, heads, dk, dv)
  if (kpt <= 2) MS_GLA_GO(2);
  if (kpt <= 4) MS_GLA_GO(4);
  if (kpt <= 6) MS_GLA_GO(6);
  if (kpt <= 8) MS_GLA_GO(8);
  if (kpt <= 12) MS_GLA_GO(12);
  MS_GLA_GO(16);
#undef MS_GLA_GO
}

template <typename TO>
__global__ void __launch_bounds__(128)
gla_output_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg, const float* __restrict__ w, float eps,
                  TO* __restrict__ out, int heads, int dv, int items) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int t = item / heads, h = item - t * heads;
  const float* x = o + (size_t)t * ldo + (size_t)h * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss += x[d] * x[d];
  ss = ms_warp_sum(ss);
  const float inv = rsqrtf(ss / (float)dv + eps);
  const float* gr = gate ? gate + (size_t)t * ldg + (size_t)h * dv : nullptr;
  for (int d = lane; d < dv; d += 32) {
    float y = x[d] * inv * (w ? w[d] : 1.f);
    if (gr) {
      const float z = gr[d];
      y *= z / (1.f + expf(-z));
    }
    out[((size_t)t * heads + h) * dv + d] = ms_from_float<TO>(y);
  }
}

// o float32 rows of heads*dv with stride ldo; gate float32 rows with stride ldg (the gate's columns begin at the pointer), or null; w float32 [dv].
MS_API int ms_gla_output(const float* o, int ldo, const float* gate, int ldg, const float* w, float eps, void* out, int out_dtype, int tokens,
                         int heads, int dv, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && heads > 0 && dv > 0 && ldo >= heads * dv && (gate == nullptr || ldg >= heads * dv), "gla_output: bad sizes");
  const int items = tokens * heads;
  const dim3 grid((items + 3) / 4), block(128);
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("gla_output", ms_launch(gla_output_kernel<float>, grid, block, 0, stream, 1, true, o, ldo, gate, ldg, w, eps, (float*)out, heads,
                                             dv, items));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("gla_output", ms_launch(gla_output_kernel<__nv_bfloat16>, grid, block, 0, stream, 1, true, o, ldo, gate, ldg, w, eps,
                                             (__nv_bfloat16*)out, heads, dv, items));
  else
    MS_REQUIRE(false, "gla_output: unknown out dtype %d", out_dtype);
  return 0;
}
