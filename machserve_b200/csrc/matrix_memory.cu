// A matrix memory with exponential gates and a running maximum (the mLSTM cell): a recurrent mixer with a matrix state,
// a normalizer vector and a stabilizer per head.
//
//   i_t = cap * tanh(x_i / cap),   f_t = logsigmoid(cap * tanh(x_f / cap))       the gates' logarithms, one number a head
//   m_t = max(f_t + m_(t-1), i_t)                                                 m_0 = 0
//   a_t = exp(f_t + m_(t-1) - m_t),   b_t = exp(i_t - m_t)
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,   n_t = a_t n_(t-1) + b_t k_t              S: [dk, dv], n: [dk], zero at the start
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//   y_t = o_t / rms(o_t) (per head, over dv, eps inside the root) * w * sigmoid(gate_t)
// Everything here is float32.
//
// A request's slot holds, per head, the matrix with the normalizer as one more column ([heads, dk, dv + 1]: n is the
// state of a value that is always 1) and, behind all matrices, the heads' m.
//
// mm_gates:   a block owns one head of one sequence.  1,024 rows at a time: the threads make the two gates of their rows, one
//             thread walks the chain m (an add and a max a row, in the rows' order, so that m does not depend on how the
//             sequence was cut), the threads make a_t and b_t of their rows from the two m beside them.  Leaves [a, b, m, 0]
//             per (row, head) and the slot's new m.
// mm_scan:    a block owns 32 (or 8) columns of [S | n] of one head of one sequence and goes through the sequence's rows of
//             the step in order, from the state the step found to the state it leaves.  Thread (c, g) holds KPT consecutive
//             key rows of column c in registers; q, k, a and b of TB rows at a time are staged in shared memory, the next
//             batch on its way while this one is worked on; the partial sums of the sixteen row groups are added in group
//             order.  Column dv comes out as n_t . q_t.  The arithmetic of a row depends on the rows before it alone, not
//             on how the sequence was cut into steps or on what else is in the batch.
// mm_output:  the division, the norm over a head's dv outputs, the weight and the gate; one warp a (row, head).
#include "launch.cuh"

#define MM_GROUPS 16
#define MM_TB 16
#define MM_CHUNK 1024
#define MM_GATE_THREADS 128

__global__ void __launch_bounds__(MM_GATE_THREADS)
mm_gates_kernel(const float* __restrict__ proj, int ld, int i_off, int f_off, const float* __restrict__ bias_i,
                const float* __restrict__ bias_f, float cap, float* __restrict__ state, long long slot_stride, long long m_off,
                const int* __restrict__ cu_tokens, const int* __restrict__ state_slots, const int* __restrict__ slot_of_token,
                float* __restrict__ gates, int heads) {
  __shared__ __align__(16) float si[MM_CHUNK], sf[MM_CHUNK], sm[MM_CHUNK + 4];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int row0 = cu_tokens[seq], rows = cu_tokens[seq + 1] - row0;
  if (rows <= 0 || slot_of_token[row0] < 0) return;
  float* mp = state + (size_t)state_slots[seq] * slot_stride + m_off + h;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv_cap = 1.f / cap;
  float m = threadIdx.x == 0 ? *mp : 0.f;
  for (int t0 = 0; t0 < rows; t0 += MM_CHUNK) {
    const int nt = min(MM_CHUNK, rows - t0);
    float xi[MM_CHUNK / MM_GATE_THREADS], xf[MM_CHUNK / MM_GATE_THREADS];
#pragma unroll
    for (int u = 0; u < MM_CHUNK / MM_GATE_THREADS; ++u) {  // every load of the round is requested before the first is used
      const int j = threadIdx.x + u * MM_GATE_THREADS;
      const float* r = proj + (size_t)(row0 + t0 + (j < nt ? j : 0)) * ld;
      xi[u] = r[i_off + h];
      xf[u] = r[f_off + h];
    }
#pragma unroll
    for (int u = 0; u < MM_CHUNK / MM_GATE_THREADS; ++u) {
      const int j = threadIdx.x + u * MM_GATE_THREADS;
      if (j < nt) {
        si[j] = cap * tanhf((xi[u] + bi) * inv_cap);
        const float z = cap * tanhf((xf[u] + bf) * inv_cap);
        sf[j] = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // the chain: an add and a max a row, in the rows' order; the loads run ahead of it
      sm[0] = m;
      int e = 0;
      for (; e + 4 <= nt; e += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(sf + e), i4 = *reinterpret_cast<const float4*>(si + e);
        const float m0 = fmaxf(f4.x + m, i4.x), m1 = fmaxf(f4.y + m0, i4.y), m2 = fmaxf(f4.z + m1, i4.z), m3 = fmaxf(f4.w + m2, i4.w);
        sm[e + 1] = m0, sm[e + 2] = m1, sm[e + 3] = m2, sm[e + 4] = m3;
        m = m3;
      }
      for (; e < nt; ++e) {
        m = fmaxf(sf[e] + m, si[e]);
        sm[e + 1] = m;
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < nt; j += MM_GATE_THREADS) {
      const float before = sm[j], now = sm[j + 1];
      float4 g;
      g.x = expf(sf[j] + before - now);
      g.y = expf(si[j] - now);
      g.z = now;
      g.w = 0.f;
      *reinterpret_cast<float4*>(gates + ((size_t)(row0 + t0 + j) * heads + h) * 4) = g;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *mp = m;
}

// proj float32 [T, ld]: the input gates' pre-activations at columns i_off + h, the forget gates' at f_off + h; biases float32
// [heads] or null; state float32, a slot every slot_stride floats, the heads' m at m_off; gates float32 [T, heads, 4].
MS_API int ms_mm_gates(const float* proj, int ld, int i_off, int f_off, const float* bias_i, const float* bias_f, float cap,
                       float* state, long long slot_stride, long long m_off, const int* cu_tokens, const int* state_slots,
                       const int* slot_of_token, float* gates, int seqs, int heads, cudaStream_t stream) {
  if (seqs == 0) return 0;
  MS_REQUIRE(seqs > 0 && heads > 0 && cap > 0.f && ld >= i_off + heads && ld >= f_off + heads && i_off >= 0 && f_off >= 0,
             "mm_gates: bad arguments seqs=%d heads=%d cap=%g ld=%d", seqs, heads, cap, ld);
  MS_REQUIRE(seqs <= 65535, "mm_gates: too many sequences for one launch");
  MS_REQUIRE(((uintptr_t)gates) % 16 == 0, "mm_gates: the gates' rows must lie on 16-byte boundaries");
  MS_LAUNCH_RESULT("mm_gates", ms_launch(mm_gates_kernel, dim3(heads, seqs), dim3(MM_GATE_THREADS), 0, stream, 1, true, proj, ld, i_off, f_off,
                                         bias_i, bias_f, cap, state, slot_stride, m_off, cu_tokens, state_slots, slot_of_token, gates,
                                         heads));
  return 0;
}

__device__ __forceinline__ void mm_cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void mm_cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// q, k, v: float32 rows of one product, row stride ld, at column offsets q_off, k_off, v_off; within each, head h begins at
// h*dk (q, k) or h*dv (v).  gates: float32 [T, heads, 4] = a, b, m, -.  state: float32, a slot every slot_stride floats, its
// head h at h*dk*(dv+1), [dk, dv+1].  o: float32 [T, heads, dv+1].  q_scale multiplies the finished sums.
template <int KPT, int COLS>
__global__ void __launch_bounds__(COLS * MM_GROUPS)
mm_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ gates, float q_scale,
               float* __restrict__ state, long long slot_stride, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
               const int* __restrict__ slot_of_token, float* __restrict__ o, int heads, int dk, int dv, int vec) {
  constexpr int KP = KPT * MM_GROUPS;           // key rows, padded
  constexpr int ROW = 2 * KP + COLS + 4;        // floats of one token in a stage: q | k | v | a b - -
  extern __shared__ __align__(16) float mm_smem[];
  float* stage0 = mm_smem;                      // [2][MM_TB][ROW]
  float* part = mm_smem + 2 * MM_TB * ROW;      // [MM_TB][MM_GROUPS][COLS]
  ms_pdl_trigger();
  ms_pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int row0 = cu_tokens[seq], rows = cu_tokens[seq + 1] - row0;
  if (rows <= 0 || slot_of_token[row0] < 0) return;  // a sequence of no rows, or rows of no request
  const int c = threadIdx.x % COLS, grp = threadIdx.x / COLS;
  const int col = c0 + c, dvn = dv + 1;
  const bool live = col < dvn;
  // padding of the key rows: q = k = 0 for good, in both stages
  for (int e = threadIdx.x; e < 2 * MM_TB * (KP - dk); e += blockDim.x) {
    const int tb = e / (KP - dk), r = dk + e % (KP - dk);
    float* t = stage0 + (size_t)tb * ROW;
    t[r] = 0.f;
    t[KP + r] = 0.f;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  auto request = [&](int t0, int st) {
    const int nt = min(MM_TB, rows - t0);
    float* base = stage0 + (size_t)st * MM_TB * ROW;
    for (int tb = warp; tb < nt; tb += nwarps) {
      const size_t t = (size_t)(row0 + t0 + tb);
      float* dst = base + (size_t)tb * ROW;
      const float* qs = proj + t * ld + q_off + h * dk;
      const float* ks = proj + t * ld + k_off + h * dk;
      const float* vs = proj + t * ld + v_off + h * dv + c0;
      if (lane == 0) mm_cp_async16(dst + 2 * KP + COLS, gates + (t * heads + h) * 4);
      if (vec) {
        for (int r = lane * 4; r < dk; r += 128) {
          mm_cp_async16(dst + r, qs + r);
          mm_cp_async16(dst + KP + r, ks + r);
        }
        for (int cc = lane * 4; cc < COLS; cc += 128) {
          if (c0 + cc < dv) mm_cp_async16(dst + 2 * KP + cc, vs + cc);  // (dv is a multiple of 4 here)
          else *reinterpret_cast<float4*>(dst + 2 * KP + cc) = make_float4(c0 + cc == dv ? 1.f : 0.f, 0.f, 0.f, 0.f);
        }
      } else {
        for (int r = lane; r < dk; r += 32) {
          mm_cp_async4(dst + r, qs + r);
          mm_cp_async4(dst + KP + r, ks + r);
        }
        for (int cc = lane; cc < COLS; cc += 32) {
          if (c0 + cc < dv) mm_cp_async4(dst + 2 * KP + cc, vs + cc);
          else dst[2 * KP + cc] = c0 + cc == dv ? 1.f : 0.f;  // the normalizer's value is 1
        }
      }
    }
  };
  request(0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  float* st = state + (size_t)state_slots[seq] * slot_stride + ((size_t)h * dk) * dvn;
  float s[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = grp * KPT + i;
    s[i] = (live && r < dk) ? st[(size_t)r * dvn + col] : 0.f;
  }
  int stg = 0;
  for (int t0 = 0; t0 < rows; t0 += MM_TB, stg ^= 1) {
    const int nt = min(MM_TB, rows - t0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // the batch has landed for every thread; the batch before has been read and its partial sums added up
    if (t0 + MM_TB < rows) request(t0 + MM_TB, stg ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    float* base = stage0 + (size_t)stg * MM_TB * ROW;
    auto token = [&](int tb) {
      const float* t = base + (size_t)tb * ROW;
      const float a = t[2 * KP + COLS], b = t[2 * KP + COLS + 1];
      const float bv = b * t[2 * KP + c];
      float acc0 = 0.f, acc1 = 0.f;  // two chains of sums (even and odd rows), added at the end: the order is fixed
      if constexpr (KPT % 4 == 0) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
          const float4 q = *reinterpret_cast<const float4*>(t + grp * KPT + i);
          const float4 k = *reinterpret_cast<const float4*>(t + KP + grp * KPT + i);
          s[i] = fmaf(a, s[i], k.x * bv);
          s[i + 1] = fmaf(a, s[i + 1], k.y * bv);
          s[i + 2] = fmaf(a, s[i + 2], k.z * bv);
          s[i + 3] = fmaf(a, s[i + 3], k.w * bv);
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
          s[i] = fmaf(a, s[i], k.x * bv);
          s[i + 1] = fmaf(a, s[i + 1], k.y * bv);
          acc0 = fmaf(s[i], q.x, acc0);
          acc1 = fmaf(s[i + 1], q.y, acc1);
        }
      }
      part[((size_t)tb * MM_GROUPS + grp) * COLS + c] = acc0 + acc1;
    };
    if (nt == MM_TB) {  // a full batch: unrolled, so that the loads of later tokens are on their way under the sums of earlier ones
#pragma unroll
      for (int tb = 0; tb < MM_TB; ++tb) token(tb);
    } else {
      for (int tb = 0; tb < nt; ++tb) token(tb);
    }
    __syncthreads();
    for (int tb = grp; tb < nt; tb += MM_GROUPS) {
      float sum = 0.f;
#pragma unroll
      for (int gi = 0; gi < MM_GROUPS; ++gi) sum += part[((size_t)tb * MM_GROUPS + gi) * COLS + c];
      if (live) o[((size_t)(row0 + t0 + tb) * heads + h) * dvn + col] = sum * q_scale;
    }
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = grp * KPT + i;
    if (live && r < dk) st[(size_t)r * dvn + col] = s[i];
  }
}

template <int KPT, int COLS>
static int mm_scan_launch(cudaStream_t stream, int seqs, const float* proj, int ld, int q_off, int k_off, int v_off, const float* gates,
                          float q_scale, float* state, long long slot_stride, const int* cu_tokens, const int* state_slots,
                          const int* slot_of_token, float* o, int heads, int dk, int dv) {
  const int vec = dk % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
                  ((uintptr_t)proj) % 16 == 0;
  constexpr int KP = KPT * MM_GROUPS;
  const size_t smem = (size_t)(2 * MM_TB * (2 * KP + COLS + 4) + MM_TB * MM_GROUPS * COLS) * sizeof(float);
  const dim3 grid((dv + 1 + COLS - 1) / COLS, heads, seqs), block(COLS * MM_GROUPS);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mm_scan_kernel<KPT, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "mm_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  MS_LAUNCH_RESULT("mm_scan", ms_launch(mm_scan_kernel<KPT, COLS>, grid, block, smem, stream, 1, true, proj, ld, q_off, k_off, v_off, gates,
                                        q_scale, state, slot_stride, cu_tokens, state_slots, slot_of_token, o, heads, dk, dv, vec));
  return 0;
}

MS_API int ms_mm_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* gates, float q_scale, float* state,
                      long long slot_stride, const int* cu_tokens, const int* state_slots, const int* slot_of_token, float* o, int seqs,
                      int heads, int dk, int dv, int narrow, cudaStream_t stream) {
  if (seqs == 0) return 0;
  MS_REQUIRE(seqs > 0 && heads > 0 && dk > 0 && dv > 0, "mm_scan: bad sizes seqs=%d heads=%d dk=%d dv=%d", seqs, heads, dk, dv);
  MS_REQUIRE(dk <= 16 * MM_GROUPS, "mm_scan: %d key channels a head are more than the kernel covers (%d)", dk, 16 * MM_GROUPS);
  MS_REQUIRE(seqs <= 65535 && heads <= 65535, "mm_scan: too many sequences or heads for one launch");
  MS_REQUIRE(((uintptr_t)gates) % 16 == 0, "mm_scan: the gates' rows must lie on 16-byte boundaries");
  const int kpt = (dk + MM_GROUPS - 1) / MM_GROUPS;
  // narrow: 8 columns a block instead of 32, for steps whose few sequences bring many rows each (the blocks of a sequence
  // are the only parallelism a scan has); a column's arithmetic is the same either way
#define MS_MM_GO(K)                                                                                                                    \
  return narrow ? mm_scan_launch<K, 8>(stream, seqs, proj, ld, q_off, k_off, v_off, gates, q_scale, state, slot_stride, cu_tokens,     \
                                       state_slots, slot_of_token, o, heads, dk, dv)                                                   \
                : mm_scan_launch<K, 32>(stream, seqs, proj, ld, q_off, k_off, v_off, gates, q_scale, state, slot_stride, cu_tokens,    \
                                        state_slots, slot_of_token, o, heads, dk, dv)
  if (kpt <= 2) MS_MM_GO(2);
  if (kpt <= 4) MS_MM_GO(4);
  if (kpt <= 6) MS_MM_GO(6);
  if (kpt <= 8) MS_MM_GO(8);
  if (kpt <= 12) MS_MM_GO(12);
  MS_MM_GO(16);
#undef MS_MM_GO
}

template <typename TO>
__global__ void __launch_bounds__(128)
mm_output_kernel(const float* __restrict__ o, const float* __restrict__ gates, const float* __restrict__ gate, int ldg,
                 const float* __restrict__ w, float eps, TO* __restrict__ out, int heads, int dv, int items) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const int t = item / heads, h = item - t * heads;
  const float* x = o + (size_t)item * (dv + 1);
  const float inv_den = 1.f / (fmaxf(fabsf(x[dv]), expf(-gates[(size_t)item * 4 + 2])) + 1e-6f);  // one division a (row, head)
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float y = x[d] * inv_den;
    ss += y * y;
  }
  ss = ms_warp_sum(ss);
  const float inv = inv_den / sqrtf(ss / (float)dv + eps);
  const float* gr = gate ? gate + (size_t)t * ldg + (size_t)h * dv : nullptr;
  for (int d = lane; d < dv; d += 32) {
    float y = x[d] * inv * (w ? w[(size_t)h * dv + d] : 1.f);
    if (gr) y *= 1.f / (1.f + expf(-gr[d]));
    out[((size_t)t * heads + h) * dv + d] = ms_from_float<TO>(y);
  }
}

// o float32 [T, heads, dv+1] (column dv: n . q); gates float32 [T, heads, 4] (m third); gate float32 rows with stride ldg (the
// gate's columns begin at the pointer), or null; w float32 [heads*dv] or null; out [T, heads*dv].
MS_API int ms_mm_output(const float* o, const float* gates, const float* gate, int ldg, const float* w, float eps, void* out,
                        int out_dtype, int tokens, int heads, int dv, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && heads > 0 && dv > 0 && (gate == nullptr || ldg >= heads * dv), "mm_output: bad sizes");
  const int items = tokens * heads;
  const dim3 grid((items + 3) / 4), block(128);
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("mm_output", ms_launch(mm_output_kernel<float>, grid, block, 0, stream, 1, true, o, gates, gate, ldg, w, eps,
                                            (float*)out, heads, dv, items));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("mm_output", ms_launch(mm_output_kernel<__nv_bfloat16>, grid, block, 0, stream, 1, true, o, gates, gate, ldg, w, eps,
                                            (__nv_bfloat16*)out, heads, dv, items));
  else
    MS_REQUIRE(false, "mm_output: unknown out dtype %d", out_dtype);
  return 0;
}
