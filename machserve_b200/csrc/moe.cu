// A routed feed-forward (mixture of experts): the router's choice, and the experts' products for (token, expert) pairs.
//
//   route:    of a token's E router logits (float32, plus the router's bias) the `top` largest are chosen (the lower index wins a tie); their
//             weights are the softmax over the chosen logits only.  ids int32 [T, top], weights float32 [T, top], in
//             descending order of the logits.  One warp a token.
//   route_scored: the other way to choose: scores s = sigmoid(logit); an expert is chosen by s + correction (a learned
//             number per expert that enters the choice only), among the experts of the best `keep` of `count` equal groups
//             of neighbours (a group's score: the sum of its two largest choice scores; the rest count as minus infinity);
//             the weights are the chosen experts' s over their sum (+ 1e-20), times `scale`.  One warp a token.
//   gate_up:  h[p, n] = act(Wg[e_p][n, :] . x[t_p, :]) * (Wu[e_p][n, :] . x[t_p, :]) for pair p = (token t_p, its j-th expert e_p)
//   down:     y[t, n] = sum_j weight[t, j] * (Wd[e_(t,j)][n, :] . h[(t, j), :]), j ascending
// The pair kernels stream the chosen experts' weights once per pair: what decoding rows want (a token reads only
// its experts) and what the 32-bit path uses for every step: each output is a chain of float32 sums whose order
// depends on the sizes alone, so a token's result does not depend on the batch.  Expert weights are stacked:
// Wg, Wu [E, ff, d], Wd [E, d, ff].  Rows of no request (slot < 0) are skipped and get zeros.
#include "launch.cuh"

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int experts, int top, int* __restrict__ ids,
                 float* __restrict__ weights, int tokens) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float* z = logits + (size_t)t * experts;
  // each lane's logits are re-read per round; an expert already chosen is passed over by comparing with the last choice
  float last_v = INFINITY;
  int last_i = -1;
  float first_v = 0.f, sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e] + (bias ? bias[e] : 0.f);
      // after (last_v, last_i) in the order: larger value first, lower index first among equals
      const bool after = v < last_v || (v == last_v && e > last_i);
      if (after && (v > best || (v == best && e < best_i))) {
        best = v;
        best_i = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (j == 0) first_v = best;
    const float w = expf(best - first_v);  // the first is the largest
    sum += w;
    if (lane == 0) {
      ids[(size_t)t * top + j] = best_i;
      weights[(size_t)t * top + j] = w;
    }
    last_v = best;
    last_i = best_i;
  }
  __syncwarp();
  if (lane == 0)
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] /= sum;
}

// logits float32 [tokens, experts]; bias float32 [experts] or null (added to the logits before the choice)
MS_API int ms_moe_route(const float* logits, const float* bias, int experts, int top, int* ids, float* weights, int tokens,
                        cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && experts > 0 && top > 0 && top <= experts, "moe_route: bad arguments tokens=%d experts=%d top=%d", tokens, experts, top);
  MS_LAUNCH_RESULT("moe_route", ms_launch(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, 1, true, logits, bias, experts, top,
                                          ids, weights, tokens));
  return 0;
}

// One warp a token; per warp in shared memory: the choice scores [experts], the groups' scores [count].
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int experts, int top, int count, int keep,
                        float scale, int* __restrict__ ids, float* __restrict__ weights, int tokens) {
  extern __shared__ float mr_smem[];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* choice = mr_smem + (size_t)warp * (experts + count);
  float* gscore = choice + experts;
  const float* z = logits + (size_t)t * experts;
  for (int e = lane; e < experts; e += 32) choice[e] = 1.f / (1.f + expf(-z[e])) + (correction ? correction[e] : 0.f);
  __syncwarp();
  const int per = experts / count;
  if (keep < count) {
    for (int g = lane; g < count; g += 32) {  // the sum of the group's two largest choice scores
      float a = -INFINITY, b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = choice[e];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // a group is kept if fewer than `keep` groups come before it in the order (larger score first, lower index first among equals)
    for (int g = lane; g < count; g += 32) {
      const float v = gscore[g];
      int before = 0;
      for (int o = 0; o < count; ++o) before += gscore[o] > v || (gscore[o] == v && o < g);
      if (before >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  float last_v = INFINITY, sum = 0.f;
  int last_i = -1;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = choice[e];
      const bool after = v < last_v || (v == last_v && e > last_i);
      if (after && (v > best || (v == best && e < best_i))) {
        best = v;
        best_i = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (best_i >= experts) best_i = 0;  // (fewer experts are allowed than a token is to choose: checked on the host)
    const float w = 1.f / (1.f + expf(-z[best_i]));  // the weight is the score without the correction
    sum += w;
    if (lane == 0) {
      ids[(size_t)t * top + j] = best_i;
      weights[(size_t)t * top + j] = w;
    }
    last_v = best;
    last_i = best_i;
  }
  __syncwarp();
  if (lane == 0)
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] = weights[(size_t)t * top + j] / (sum + 1e-20f) * scale;
}

// logits float32 [tokens, experts]; correction float32 [experts] or null; count groups of experts / count neighbours, keep of them
MS_API int ms_moe_route_scored(const float* logits, const float* correction, int experts, int top, int count, int keep, float scale,
                               int* ids, float* weights, int tokens, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && experts > 0 && top > 0 && count > 0 && keep > 0 && keep <= count && experts % count == 0,
             "moe_route_scored: bad arguments tokens=%d experts=%d top=%d groups=%d keep=%d", tokens, experts, top, count, keep);
  MS_REQUIRE(top <= experts / count * keep, "moe_route_scored: %d experts a token, but only %d are in the %d kept groups", top,
             experts / count * keep, keep);
  const size_t smem = (size_t)4 * (experts + count) * sizeof(float);
  MS_REQUIRE(smem <= 48 * 1024, "moe_route_scored: %d experts are more than the kernel covers", experts);
  MS_LAUNCH_RESULT("moe_route_scored", ms_launch(moe_route_scored_kernel, dim3((tokens + 3) / 4), dim3(128), smem, stream, 1, true, logits,
                                                 correction, experts, top, count, keep, scale, ids, weights, tokens));
  return 0;
}

__device__ __forceinline__ float moe_act(float g, int act) {
  if (act == 0) return g / (1.f + expf(-g));
  if (act == 2) return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));  // the exact GELU
  return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

#define MOE_WARPS 8

// eight consecutive weights (16 bytes of bfloat16, 32 of float32) times eight floats of shared memory, added to s in order
__device__ __forceinline__ float moe_dot8(const float* w, const float* x, float s) {
  const float4 a = *reinterpret_cast<const float4*>(w), b = *reinterpret_cast<const float4*>(w + 4);
  const float4 p = *reinterpret_cast<const float4*>(x), q = *reinterpret_cast<const float4*>(x + 4);
  s = fmaf(a.x, p.x, s); s = fmaf(a.y, p.y, s); s = fmaf(a.z, p.z, s); s = fmaf(a.w, p.w, s);
  s = fmaf(b.x, q.x, s); s = fmaf(b.y, q.y, s); s = fmaf(b.z, q.z, s); s = fmaf(b.w, q.w, s);
  return s;
}
__device__ __forceinline__ float moe_dot8(const __nv_bfloat16* w, const float* x, float s) {
  const uint4 u = *reinterpret_cast<const uint4*>(w);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float4 p = *reinterpret_cast<const float4*>(x), q = *reinterpret_cast<const float4*>(x + 4);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
  s = fmaf(a.x, p.x, s); s = fmaf(a.y, p.y, s); s = fmaf(b.x, p.z, s); s = fmaf(b.y, p.w, s);
  s = fmaf(c.x, q.x, s); s = fmaf(c.y, q.y, s); s = fmaf(d.x, q.z, s); s = fmaf(d.y, q.w, s);
  return s;
}

// grid (ceil(ff / MOE_WARPS), pairs); a warp an output column; x row of the pair's token in shared memory as float32
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_gate_up_pairs_kernel(const T* __restrict__ x, const T* __restrict__ wg, const T* __restrict__ wu, const int* __restrict__ ids,
                         const int* __restrict__ slots, T* __restrict__ h, int top, int d, int ff, int experts, int act, int vec) {
  extern __shared__ __align__(16) float moe_x[];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int pair = blockIdx.y, t = pair / top;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * MOE_WARPS + warp;
  if (slots[t] < 0) {
    if (n < ff && lane == 0) h[(size_t)pair * ff + n] = ms_from_float<T>(0.f);
    return;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) moe_x[c] = ms_to_float(x[(size_t)t * d + c]);
  __syncthreads();
  if (n >= ff) return;
  int e = ids[pair];
  e = e < 0 ? 0 : (e >= experts ? experts - 1 : e);
  const T* g = wg + ((size_t)e * ff + n) * d;
  const T* u = wu ? wu + ((size_t)e * ff + n) * d : nullptr;  // (no second matrix: experts without a gate, h = act(Wg x))
  float sg = 0.f, su = 0.f;
  if (vec) {  // (the order of a sum depends on d and on this flag, which depends on d and the pointers' alignment alone)
    for (int c = lane * 8; c < d; c += 256) {
      sg = moe_dot8(g + c, moe_x + c, sg);
      if (u) su = moe_dot8(u + c, moe_x + c, su);
    }
  } else {
    for (int c = lane; c < d; c += 32) {
      const float xv = moe_x[c];
      sg = fmaf(ms_to_float(g[c]), xv, sg);
      if (u) su = fmaf(ms_to_float(u[c]), xv, su);
    }
  }
  sg = ms_warp_sum(sg);
  su = u ? ms_warp_sum(su) : 1.f;
  if (lane == 0) h[(size_t)pair * ff + n] = ms_from_float<T>(moe_act(sg, act) * su);
}

// grid (ceil(d / MOE_WARPS), tokens); a warp an output column, the token's experts in turn
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_pairs_kernel(const T* __restrict__ h, const T* __restrict__ wd, const int* __restrict__ ids, const float* __restrict__ weights,
                      const int* __restrict__ slots, float* __restrict__ y, int top, int d, int ff, int experts, int vec) {
  extern __shared__ __align__(16) float moe_h[];  // [top][ff]
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * MOE_WARPS + warp;
  if (slots[t] < 0) {
    if (n < d && lane == 0) y[(size_t)t * d + n] = 0.f;
    return;
  }
  for (int c = threadIdx.x; c < top * ff; c += blockDim.x) moe_h[c] = ms_to_float(h[(size_t)t * top * ff + c]);
  __syncthreads();
  if (n >= d) return;
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    int e = ids[(size_t)t * top + j];
    e = e < 0 ? 0 : (e >= experts ? experts - 1 : e);
    const T* w = wd + ((size_t)e * d + n) * ff;
    const float* hj = moe_h + (size_t)j * ff;
    float s = 0.f;
    if (vec) {
      for (int c = lane * 8; c < ff; c += 256) s = moe_dot8(w + c, hj + c, s);
    } else {
      for (int c = lane; c < ff; c += 32) s = fmaf(ms_to_float(w[c]), hj[c], s);
    }
    s = ms_warp_sum(s);
    total = fmaf(weights[(size_t)t * top + j], s, total);
  }
  if (lane == 0) y[(size_t)t * d + n] = total;
}

// x [T, d], h [T*top, ff] in the weights' type (dtype); y float32 [T, d].
MS_API int ms_moe_gate_up_pairs(const void* x, const void* wg, const void* wu, const int* ids, const int* slots, void* h, int dtype,
                                int tokens, int top, int d, int ff, int experts, int act, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && top > 0 && d > 0 && ff > 0 && experts > 0 && act >= 0 && act <= 2, "moe_gate_up_pairs: bad arguments");
  MS_REQUIRE((long long)tokens * top <= 65535, "moe_gate_up_pairs: %d pairs are more than one launch takes", tokens * top);
  MS_REQUIRE((size_t)d * 4 <= 48 * 1024, "moe_gate_up_pairs: rows of %d are too wide", d);
  const dim3 grid((ff + MOE_WARPS - 1) / MOE_WARPS, tokens * top), block(MOE_WARPS * 32);
  const int vec = d % 8 == 0 && ((uintptr_t)wg | (uintptr_t)wu) % 32 == 0;  // (wu may be null: experts without a gate)
  if (dtype == MS_F32)
    MS_LAUNCH_RESULT("moe_gate_up_pairs", ms_launch(moe_gate_up_pairs_kernel<float>, grid, block, (size_t)d * 4, stream, 1, true, (const float*)x,
                                                    (const float*)wg, (const float*)wu, ids, slots, (float*)h, top, d, ff, experts, act, vec));
  else if (dtype == MS_BF16)
    MS_LAUNCH_RESULT("moe_gate_up_pairs",
                     ms_launch(moe_gate_up_pairs_kernel<__nv_bfloat16>, grid, block, (size_t)d * 4, stream, 1, true, (const __nv_bfloat16*)x,
                               (const __nv_bfloat16*)wg, (const __nv_bfloat16*)wu, ids, slots, (__nv_bfloat16*)h, top, d, ff, experts, act, vec));
  else
    MS_REQUIRE(false, "moe_gate_up_pairs: unknown dtype %d", dtype);
  return 0;
}

MS_API int ms_moe_down_pairs(const void* h, const void* wd, const int* ids, const float* weights, const int* slots, float* y, int dtype,
                             int tokens, int top, int d, int ff, int experts, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && top > 0 && d > 0 && ff > 0 && experts > 0, "moe_down_pairs: bad arguments");
  MS_REQUIRE(tokens <= 65535, "moe_down_pairs: %d tokens are more than one launch takes", tokens);
  const size_t smem = (size_t)top * ff * 4;
  MS_REQUIRE(smem <= 200 * 1024, "moe_down_pairs: %d experts of %d a token need %zu bytes of shared memory", top, ff, smem);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t e1 = cudaFuncSetAttribute(moe_down_pairs_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e2 = cudaFuncSetAttribute(moe_down_pairs_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e1 == cudaSuccess && e2 == cudaSuccess, "moe_down_pairs: cannot get %zu bytes of shared memory", smem);
    configured = smem;
  }
  const dim3 grid((d + MOE_WARPS - 1) / MOE_WARPS, tokens), block(MOE_WARPS * 32);
  const int vec = ff % 8 == 0 && (uintptr_t)wd % 32 == 0;
  if (dtype == MS_F32)
    MS_LAUNCH_RESULT("moe_down_pairs", ms_launch(moe_down_pairs_kernel<float>, grid, block, smem, stream, 1, true, (const float*)h,
                                                 (const float*)wd, ids, weights, slots, y, top, d, ff, experts, vec));
  else if (dtype == MS_BF16)
    MS_LAUNCH_RESULT("moe_down_pairs", ms_launch(moe_down_pairs_kernel<__nv_bfloat16>, grid, block, smem, stream, 1, true,
                                                 (const __nv_bfloat16*)h, (const __nv_bfloat16*)wd, ids, weights, slots, y, top, d, ff, experts, vec));
  else
    MS_REQUIRE(false, "moe_down_pairs: unknown dtype %d", dtype);
  return 0;
}
