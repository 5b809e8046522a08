// The gated delta rule: a recurrent mixer with a matrix state per head that is decayed, corrected towards the new value and
// read, token by token; its inputs pass a short causal convolution over time first.
//
//   x_t = [q | k | v] (G*dk, G*dk, H*dv channels) of the token's input product, float32
//   y_t[c] = silu(sum_j w[c, j] * x_(t - (taps-1) + j)[c])        (zeros before the start of the sequence; the last taps - 1
//                                                                   inputs of a sequence are part of its state)
//   q, k: every head divided by sqrt(sum of its squares + 1e-6); q also times q_scale
//   beta_t[h] = sigmoid(b_t[h]);   g_t[h] = exp(-exp(A_log[h]) * softplus(a_t[h] + dt_bias[h]))
//   per value head h (reading q/k head h / (H / G)), S [dk, dv] float32, zero at the start of a sequence:
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// Everything here is float32.
//
// gdr_prepare:      a block a token: the convolution and SiLU of its C channels, the unit vectors, beta and g.
// gdr_conv_update:  a thread a (sequence, channel): the state's last taps - 1 inputs after the step's rows.
// gdr_scan:         a block owns COLS value columns of one head of one sequence and goes through the sequence's rows of the step
//                   in order, from the state the step found to the state it leaves.  Eight lanes share a column: lane (c, g)
//                   holds KPT key rows of column c in registers, W (4, or 2) neighbours out of every 8 W, so that the eight
//                   lanes of a column read a staged q or k with loads that lie side by side.  With a = k . S_old[:, c], b = q . S_old[:, c] and
//                   qk = q . k (three sums over the eight lanes, by exchange within the warp, every lane the same bits):
//                     u = beta (v - g a),  o = g b + qk u,  S[:, c] <- g S[:, c] + k u.
//                   q, k, v, beta and g of 16 tokens at a time are staged in shared memory, the next batch on its way while
//                   this one is worked on.  A token's arithmetic depends on the tokens before it alone, not on how the
//                   sequence was cut into steps or on what else is in the batch.
// A request's state is one row of `state` (float32, `stride` floats a slot): the matrices [H, dk, dv] first, then, from
// `conv_off` on, the last taps - 1 inputs [taps - 1, C], oldest first.
#include "launch.cuh"

#define GDR_LPC 8     // lanes that share a value column
#define GDR_TB 16     // tokens of a staged batch
#define GDR_MAX_TAPS 16

__device__ __forceinline__ float gdr_silu(float z) { return z / (1.f + expf(-z)); }

__global__ void __launch_bounds__(256)
gdr_prepare_kernel(const float* __restrict__ proj, int ld, int x_off, int b_off, int a_off, const float* __restrict__ conv_w, int taps,
                   const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ state, long long stride,
                   long long conv_off, const int* __restrict__ cu_tokens, const int* __restrict__ seq_of_token,
                   const int* __restrict__ slot_of_token, float* __restrict__ qkv, float* __restrict__ bg, int heads, int groups, int dk,
                   int dv, float q_scale) {
  extern __shared__ float gdr_y[];  // [C]
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int slot = slot_of_token[t];
  if (slot < 0) return;
  const int i = t - cu_tokens[seq_of_token[t]];  // rows of this sequence that the step brings before this one
  const int C = 2 * groups * dk + heads * dv, K = taps - 1;
  const float* old = state + (size_t)slot * stride + conv_off;  // [K, C], oldest first
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < taps; ++j) {  // oldest first: lag K - j
      const int lag = K - j;
      const float x = lag <= i ? proj[(size_t)(t - lag) * ld + x_off + c] : old[(size_t)(K - (lag - i)) * C + c];
      s = fmaf(conv_w[(size_t)c * taps + j], x, s);
    }
    gdr_y[c] = gdr_silu(s);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* out = qkv + (size_t)t * C;
  for (int h = warp; h < 2 * groups; h += nwarps) {  // the q heads, then the k heads
    const float* y = gdr_y + h * dk;
    float ss = 0.f;
    for (int e = lane; e < dk; e += 32) ss = fmaf(y[e], y[e], ss);
    ss = ms_warp_sum(ss);
    const float inv = (h < groups ? q_scale : 1.f) / sqrtf(ss + 1e-6f);
    for (int e = lane; e < dk; e += 32) out[h * dk + e] = y[e] * inv;
  }
  for (int c = 2 * groups * dk + threadIdx.x; c < C; c += blockDim.x) out[c] = gdr_y[c];
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float b = proj[(size_t)t * ld + b_off + h];
    const float z = proj[(size_t)t * ld + a_off + h] + dt_bias[h];
    const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
    bg[(size_t)t * 2 * heads + h] = 1.f / (1.f + expf(-b));
    bg[(size_t)t * 2 * heads + heads + h] = expf(-expf(a_log[h]) * sp);
  }
}

__global__ void gdr_conv_update_kernel(const float* __restrict__ proj, int ld, int x_off, int taps, float* __restrict__ state,
                                       long long stride, long long conv_off, const int* __restrict__ cu_tokens,
                                       const int* __restrict__ state_slots, const int* __restrict__ slot_of_token, int C) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int seq = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row0 = cu_tokens[seq], n = cu_tokens[seq + 1] - row0;
  if (n <= 0 || slot_of_token[row0] < 0) return;
  const int K = taps - 1;
  float* st = state + (size_t)state_slots[seq] * stride + conv_off;
  // place j of the new state is input n + j of (the K old inputs, then the step's n): read ahead of every write
  for (int j = 0; j < K; ++j) {
    const int idx = n + j;
    st[(size_t)j * C + c] = idx < K ? st[(size_t)idx * C + c] : proj[(size_t)(row0 + idx - K) * ld + x_off + c];
  }
}

__device__ __forceinline__ void gdr_cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void gdr_cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

template <int KPT, int COLS>
__global__ void __launch_bounds__(COLS * GDR_LPC + (COLS == 8 ? 32 : 0), (COLS == 32 && KPT <= 16) ? 2 : 1)
gdr_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ bg, float* __restrict__ state, long long stride,
                const int* __restrict__ cu_tokens, const int* __restrict__ state_slots, const int* __restrict__ slot_of_token,
                float* __restrict__ o, int heads, int groups, int dk, int dv, int vec) {
  constexpr int KP = KPT * GDR_LPC;       // key rows, padded
  constexpr int ROW = 2 * KP + COLS + 4;  // floats of one token in a stage: q | k | v | beta, g, -, -
  constexpr int W = KPT % 4 == 0 ? 4 : 2;  // key rows that a lane reads with one load (KPT is a multiple of 2)
  extern __shared__ __align__(16) float gdr_smem[];
  float* stage0 = gdr_smem;                       // [2][GDR_TB][ROW]
  float* obuf = gdr_smem + 2 * GDR_TB * ROW;      // [GDR_TB][COLS]
  ms_pdl_trigger();
  ms_pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int row0 = cu_tokens[seq], rows = cu_tokens[seq + 1] - row0;
  if (rows <= 0 || slot_of_token[row0] < 0) return;  // a sequence of no rows, or rows of no request
  const int slot = state_slots[seq];
  // blocks of few columns (long portions) have one warp more, which does nothing but request the batches: the lanes that
  // walk the chain of tokens spend no instruction on it
  constexpr bool FEEDER = COLS == 8;
  const bool feeds = FEEDER && threadIdx.x >= COLS * GDR_LPC;
  const int grp = threadIdx.x % GDR_LPC, c = feeds ? 0 : threadIdx.x / GDR_LPC;  // (the lanes of a column are neighbours in a warp)
  const int col = c0 + c;
  const bool live = !feeds && col < dv;
  const int qh = h / (heads / groups);
  const int C = 2 * groups * dk + heads * dv;
  // padding of the key rows: q = k = 0 for good, in both stages
  for (int e = threadIdx.x; e < 2 * GDR_TB * (KP - dk); e += blockDim.x) {
    const int tb = e / (KP - dk), r = dk + e % (KP - dk);
    float* t = stage0 + (size_t)tb * ROW;
    t[r] = 0.f;
    t[KP + r] = 0.f;
  }
  const int lane = threadIdx.x & 31, warp = FEEDER ? 0 : threadIdx.x >> 5, nwarps = FEEDER ? 1 : blockDim.x >> 5;
  auto request = [&](int t0, int st) {
    if (FEEDER && !feeds) return;
    const int nt = min(GDR_TB, rows - t0);
    float* base = stage0 + (size_t)st * GDR_TB * ROW;
    for (int tb = warp; tb < nt; tb += nwarps) {
      const size_t t = (size_t)(row0 + t0 + tb);
      float* dst = base + (size_t)tb * ROW;
      const float* qs = qkv + t * C + qh * dk;
      const float* ks = qkv + t * C + groups * dk + qh * dk;
      const float* vs = qkv + t * C + 2 * groups * dk + h * dv + c0;
      if (vec) {
        for (int r = lane * 4; r < dk; r += 128) {
          gdr_cp_async16(dst + r, qs + r);
          gdr_cp_async16(dst + KP + r, ks + r);
        }
        for (int cc = lane * 4; cc < COLS; cc += 128) {
          if (c0 + cc < dv) gdr_cp_async16(dst + 2 * KP + cc, vs + cc);  // (dv is a multiple of 4 here)
          else *reinterpret_cast<float4*>(dst + 2 * KP + cc) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
        for (int r = lane; r < dk; r += 32) {
          gdr_cp_async4(dst + r, qs + r);
          gdr_cp_async4(dst + KP + r, ks + r);
        }
        for (int cc = lane; cc < COLS; cc += 32) {
          if (c0 + cc < dv) gdr_cp_async4(dst + 2 * KP + cc, vs + cc);
          else dst[2 * KP + cc] = 0.f;
        }
      }
      if (lane < 2) gdr_cp_async4(dst + 2 * KP + COLS + lane, bg + t * 2 * heads + lane * heads + h);
    }
  };
  request(0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  float* st = state + (size_t)slot * stride + ((size_t)h * dk) * dv;
  float s[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = (i / W) * (GDR_LPC * W) + grp * W + i % W;
    s[i] = (live && r < dk) ? st[(size_t)r * dv + col] : 0.f;
  }
  // one token's inputs in registers: this lane's key rows of q and k, the column's v, the head's beta and g
  struct Tok {
    float q[KPT], k[KPT], v, beta, g;
  };
  auto fetch = [&](const float* t, Tok& x) {  // loads and nothing that waits for them: a warp issues in order
    x.v = t[2 * KP + c];
    x.beta = t[2 * KP + COLS];
    x.g = t[2 * KP + COLS + 1];
#pragma unroll
    for (int i = 0; i < KPT; i += W) {
      const int at = (i / W) * (GDR_LPC * W) + grp * W;
      if constexpr (W == 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(t + at);
        const float4 k4 = *reinterpret_cast<const float4*>(t + KP + at);
        x.q[i] = q4.x; x.q[i + 1] = q4.y; x.q[i + 2] = q4.z; x.q[i + 3] = q4.w;
        x.k[i] = k4.x; x.k[i + 1] = k4.y; x.k[i + 2] = k4.z; x.k[i + 3] = k4.w;
      } else {
        const float2 q2 = *reinterpret_cast<const float2*>(t + at);
        const float2 k2 = *reinterpret_cast<const float2*>(t + KP + at);
        x.q[i] = q2.x; x.q[i + 1] = q2.y;
        x.k[i] = k2.x; x.k[i + 1] = k2.y;
      }
    }
  };
  auto work = [&](const Tok& x, int tb) {
    float pa[W], pb[W], pq[W];
#pragma unroll
    for (int j = 0; j < W; ++j) pa[j] = pb[j] = pq[j] = 0.f;
#pragma unroll
    for (int i = 0; i < KPT; ++i) pa[i % W] = fmaf(x.k[i], s[i], pa[i % W]);  // (the sum that the state's next value waits for)
#pragma unroll
    for (int i = 0; i < KPT; ++i) {  // W sums side by side, so that a lane's chain of additions is KPT / W long
      pb[i % W] = fmaf(x.q[i], s[i], pb[i % W]);
      pq[i % W] = fmaf(x.q[i], x.k[i], pq[i % W]);
    }
    float a = W == 4 ? (pa[0] + pa[1]) + (pa[2] + pa[W - 1]) : pa[0] + pa[W - 1];
    float b = W == 4 ? (pb[0] + pb[1]) + (pb[2] + pb[W - 1]) : pb[0] + pb[W - 1];
    float qk = W == 4 ? (pq[0] + pq[1]) + (pq[2] + pq[W - 1]) : pq[0] + pq[W - 1];
#pragma unroll
    for (int off = 1; off < GDR_LPC; off <<= 1) {  // both lanes of a pair add the same two numbers: the same bits in every lane
      const float a2 = __shfl_xor_sync(0xffffffffu, a, off);  // three exchanges under way at once, one wait a stage
      const float b2 = __shfl_xor_sync(0xffffffffu, b, off);
      const float q2 = __shfl_xor_sync(0xffffffffu, qk, off);
      a += a2;
      b += b2;
      qk += q2;
    }
    const float u = x.beta * (x.v - x.g * a);
#pragma unroll
    for (int i = 0; i < KPT; ++i) s[i] = fmaf(x.g, s[i], x.k[i] * u);
    if (grp == 0) obuf[tb * COLS + c] = fmaf(x.g, b, qk * u);
  };
  int stg = 0;
  for (int t0 = 0; t0 < rows; t0 += GDR_TB, stg ^= 1) {
    const int nt = min(GDR_TB, rows - t0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // the batch has landed for every thread; the batch before has been read and its outputs written
    if (t0 + GDR_TB < rows) request(t0 + GDR_TB, stg ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    const float* base = stage0 + (size_t)stg * GDR_TB * ROW;
    if (feeds) {
      // (nothing between the two barriers)
    } else if constexpr (COLS == 8) {
      // blocks of few columns are for long portions: the next token's inputs are on their way while this one's chain
      // (a -> u -> S) runs
      Tok even, odd;
      fetch(base, even);
      for (int tb = 0; tb < nt; tb += 2) {
        if (tb + 1 < nt) fetch(base + (size_t)(tb + 1) * ROW, odd);
        work(even, tb);
        if (tb + 1 < nt) {
          if (tb + 2 < nt) fetch(base + (size_t)(tb + 2) * ROW, even);
          work(odd, tb + 1);
        }
      }
    } else {
      // blocks of many columns are for steps of single tokens, where the state's way from and to memory is what counts:
      // fewer registers, more blocks on a multiprocessor
      for (int tb = 0; tb < nt; ++tb) {
        Tok x;
        fetch(base + (size_t)tb * ROW, x);
        work(x, tb);
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * COLS; e += blockDim.x) {
      const int tb = e / COLS, cc = e - tb * COLS;
      if (c0 + cc < dv) o[(size_t)(row0 + t0 + tb) * ((size_t)heads * dv) + h * dv + c0 + cc] = obuf[e];
    }
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int r = (i / W) * (GDR_LPC * W) + grp * W + i % W;
    if (live && r < dk) st[(size_t)r * dv + col] = s[i];
  }
}

template <int KPT, int COLS>
static int gdr_scan_launch(cudaStream_t stream, int seqs, const float* qkv, const float* bg, float* state, long long stride,
                           const int* cu_tokens, const int* state_slots, const int* slot_of_token, float* o, int heads, int groups, int dk,
                           int dv) {
  const int C = 2 * groups * dk + heads * dv;
  const int vec = dk % 4 == 0 && dv % 4 == 0 && C % 4 == 0 && (uintptr_t)qkv % 16 == 0;
  constexpr int KP = KPT * GDR_LPC;
  const size_t smem = (size_t)(2 * GDR_TB * (2 * KP + COLS + 4) + GDR_TB * COLS) * sizeof(float);
  const dim3 grid((dv + COLS - 1) / COLS, heads, seqs), block(COLS * GDR_LPC + (COLS == 8 ? 32 : 0));
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdr_scan_kernel<KPT, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "gdr_scan: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  MS_LAUNCH_RESULT("gdr_scan", ms_launch(gdr_scan_kernel<KPT, COLS>, grid, block, smem, stream, 1, true, qkv, bg, state, stride, cu_tokens,
                                         state_slots, slot_of_token, o, heads, groups, dk, dv, vec));
  return 0;
}

// proj float32 [T, ld]: the conv channels [q | k | v] from column x_off, the heads' b from b_off and a from a_off.  conv_w float32
// [C, taps] (the last column is the current token's).  qkv float32 [T, C] and bg float32 [T, 2*heads] (beta | g) are written.
MS_API int ms_gdr_prepare(const float* proj, int ld, int x_off, int b_off, int a_off, const float* conv_w, int taps, const float* a_log,
                          const float* dt_bias, const float* state, long long stride, long long conv_off, const int* cu_tokens,
                          const int* seq_of_token, const int* slot_of_token, float* qkv, float* bg, int tokens, int heads, int groups,
                          int dk, int dv, float q_scale, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && heads > 0 && groups > 0 && dk > 0 && dv > 0 && heads % groups == 0, "gdr_prepare: bad sizes");
  MS_REQUIRE(taps >= 1 && taps <= GDR_MAX_TAPS, "gdr_prepare: %d taps are more than the kernel covers (%d)", taps, GDR_MAX_TAPS);
  const int C = 2 * groups * dk + heads * dv;
  MS_REQUIRE((size_t)C * 4 <= 48 * 1024, "gdr_prepare: %d channels are more than the kernel covers", C);
  MS_LAUNCH_RESULT("gdr_prepare", ms_launch(gdr_prepare_kernel, dim3(tokens), dim3(256), (size_t)C * 4, stream, 1, true, proj, ld, x_off, b_off,
                                            a_off, conv_w, taps, a_log, dt_bias, state, stride, conv_off, cu_tokens, seq_of_token,
                                            slot_of_token, qkv, bg, heads, groups, dk, dv, q_scale));
  return 0;
}

MS_API int ms_gdr_conv_update(const float* proj, int ld, int x_off, int taps, float* state, long long stride, long long conv_off,
                              const int* cu_tokens, const int* state_slots, const int* slot_of_token, int seqs, int channels,
                              cudaStream_t stream) {
  if (seqs == 0 || taps <= 1) return 0;
  MS_REQUIRE(seqs > 0 && seqs <= 65535 && channels > 0 && taps <= GDR_MAX_TAPS, "gdr_conv_update: bad sizes");
  MS_LAUNCH_RESULT("gdr_conv_update", ms_launch(gdr_conv_update_kernel, dim3((channels + 127) / 128, seqs), dim3(128), 0, stream, 1, true, proj,
                                                ld, x_off, taps, state, stride, conv_off, cu_tokens, state_slots, slot_of_token, channels));
  return 0;
}

// qkv, bg as gdr_prepare leaves them; state float32 rows of `stride` floats, the matrices [heads, dk, dv] first; o float32
// [T, heads*dv].  `narrow`: blocks of 8 value columns instead of 32 (more blocks a sequence: for steps with long portions);
// a column's arithmetic is the same either way.
MS_API int ms_gdr_scan(const float* qkv, const float* bg, float* state, long long stride, const int* cu_tokens, const int* state_slots,
                       const int* slot_of_token, float* o, int seqs, int heads, int groups, int dk, int dv, int narrow,
                       cudaStream_t stream) {
  if (seqs == 0) return 0;
  MS_REQUIRE(seqs > 0 && heads > 0 && groups > 0 && dk > 0 && dv > 0 && heads % groups == 0, "gdr_scan: bad sizes");
  MS_REQUIRE(dk <= 32 * GDR_LPC, "gdr_scan: %d key channels a head are more than the kernel covers (%d)", dk, 32 * GDR_LPC);
  MS_REQUIRE(seqs <= 65535 && heads <= 65535, "gdr_scan: too many sequences or heads for one launch");
  const int kpt = (dk + GDR_LPC - 1) / GDR_LPC;
#define MS_GDR_GO(K)                                                                                                               \
  return narrow ? gdr_scan_launch<K, 8>(stream, seqs, qkv, bg, state, stride, cu_tokens, state_slots, slot_of_token, o, heads,     \
                                        groups, dk, dv)                                                                            \
                : gdr_scan_launch<K, 32>(stream, seqs, qkv, bg, state, stride, cu_tokens, state_slots, slot_of_token, o, heads,    \
                                         groups, dk, dv)
  if (kpt <= 2) MS_GDR_GO(2);
  if (kpt <= 4) MS_GDR_GO(4);
  if (kpt <= 8) MS_GDR_GO(8);
  if (kpt <= 16) MS_GDR_GO(16);
  MS_GDR_GO(32);
#undef MS_GDR_GO
}
