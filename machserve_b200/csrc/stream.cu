// Kernels around the residual stream for layers whose two halves are summed before they are added, with an RMS norm:
//
// * embed_scaled_pos: x[r, :] = E[token[r], :] * scale + P[position[r], :] in float32 (P a learned table, or none);
// * add_streams_rmsnorm: x <- x + (m * (a + b) + first + vec), then, when a weight is given, out = x / rms(x) * w
//   (m: a multiplier of the deltas, 1 for most layers).
//   a, b: deltas of the step's rows (float32 or bfloat16, either may be absent); first: another float32 stream
//   [T, d] (the embedding's output, for the start of a pass over looped layers); vec: one float32 row added to
//   every row.  Without a weight the kernel only adds (the entry of a pass).  With `rows`, output row i is made
//   from input row rows[i] and nothing is written back (the final norm of the wanted rows).
//   The sums and the norm are float32; the order of a row's additions depends on d alone.
// * norm_pair_mean: out = m * (a / rms(a) * wa + b / rms(b) * wb), each rms over the row's d elements with eps inside the
//   root: the two halves of a mixer made of two, each normed with a weight of its own, in float32.
// * pair_weighted_sum: out = sa * (a + bias_a) + sb * (b + bias_b), the biases float32 [d] or absent: the two halves of a mixer
//   made of two, each with a multiplier of its own (and the bias of its output projection), in float32.
// * gated_act_mul: out[r, c] = act(gate_up[r, c]) * gate_up[r, inter + c], act = SiLU or the tanh form of GELU,
//   computed in float32 from a float32 or bfloat16 product.
#include "launch.cuh"

template <typename TW>
__global__ void embed_scaled_pos_kernel(const TW* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ positions,
                                        const float* __restrict__ pos_table, float* __restrict__ out, int d, int vocab, int max_pos,
                                        float scale) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;  // ids are checked on the host; a row of no request gets zeros
  const TW* src = table + (size_t)(ok ? id : 0) * d;
  int p = positions[row];
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
  const float* pr = pos_table ? pos_table + (size_t)p * d : nullptr;
  float* dst = out + (size_t)row * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = ok ? ms_to_float(src[c]) * scale : 0.f;
    if (pr && ok) v += pr[c];
    dst[c] = v;
  }
}

MS_API int ms_embed_scaled_pos(const void* table, int table_dtype, const int* ids, const int* positions, const float* pos_table,
                               float* out, int rows, int d, int vocab, int max_pos, float scale, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && d > 0 && vocab > 0 && (pos_table == nullptr || max_pos > 0), "embed_scaled_pos: bad sizes rows=%d d=%d vocab=%d",
             rows, d, vocab);
  const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
  if (table_dtype == MS_F32)
    MS_LAUNCH_RESULT("embed_scaled_pos", ms_launch(embed_scaled_pos_kernel<float>, dim3(rows), dim3(threads), 0, stream, 1, true,
                                                   (const float*)table, ids, positions, pos_table, out, d, vocab, max_pos, scale));
  else if (table_dtype == MS_BF16)
    MS_LAUNCH_RESULT("embed_scaled_pos", ms_launch(embed_scaled_pos_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, 1, true,
                                                   (const __nv_bfloat16*)table, ids, positions, pos_table, out, d, vocab, max_pos, scale));
  else
    MS_REQUIRE(false, "embed_scaled_pos: unknown table dtype %d", table_dtype);
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float4 st_load4(const void* p, int dtype, size_t i) {
  if (dtype == MS_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float st_load1(const void* p, int dtype, size_t i) {
  return dtype == MS_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
template <typename TO>
__device__ __forceinline__ void st_store4(TO* p, float4 v);
template <>
__device__ __forceinline__ void st_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void st_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 u;
  *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

#define ST_THREADS 256
#define ST_KEEP 8  // groups of four elements a thread keeps in registers: d <= 256 * 8 * 4

// VEC: d is a multiple of 4, every pointer 16-byte aligned (8 for bfloat16 deltas), d <= ST_THREADS * ST_KEEP * 4:
// the summed row stays in registers between the two passes.
template <typename TO, bool VEC>
__global__ void __launch_bounds__(ST_THREADS)
add_streams_rmsnorm_kernel(float* __restrict__ residual, const void* __restrict__ a, int a_dtype, const void* __restrict__ b,
                           int b_dtype, const float* __restrict__ first, const float* __restrict__ vec,
                           const float* __restrict__ weight, TO* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                           float m) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  const size_t base = (size_t)irow * d;
  const bool adds = a || b || first || vec;
  float ss = 0.f;
  if (VEC) {
    float4 v[ST_KEEP];
    const int ngroups = d / 4;
#pragma unroll
    for (int i = 0; i < ST_KEEP; ++i) {
      const int g = threadIdx.x + i * ST_THREADS;
      if (g < ngroups) {
        // every load is requested before the first is used: one round trip to memory, not one per stream
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 x = *reinterpret_cast<const float4*>(residual + base + 4 * g);
        const float4 ta = a ? st_load4(a, a_dtype, base + 4 * g) : zero;
        const float4 tb = b ? st_load4(b, b_dtype, base + 4 * g) : zero;
        const float4 tf = first ? *reinterpret_cast<const float4*>(first + base + 4 * g) : zero;
        const float4 tv = vec ? *reinterpret_cast<const float4*>(vec + 4 * g) : zero;
        float4 s = make_float4(((ta.x + tb.x) * m + tf.x) + tv.x, ((ta.y + tb.y) * m + tf.y) + tv.y, ((ta.z + tb.z) * m + tf.z) + tv.z,
                               ((ta.w + tb.w) * m + tf.w) + tv.w);
        x.x += s.x; x.y += s.y; x.z += s.z; x.w += s.w;
        if (adds && !rows) *reinterpret_cast<float4*>(residual + base + 4 * g) = x;
        v[i] = x;
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
      }
    }
    if (!weight) return;
    ss = ms_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)orow * d;
#pragma unroll
    for (int i = 0; i < ST_KEEP; ++i) {
      const int g = threadIdx.x + i * ST_THREADS;
      if (g < ngroups) {
        const float4 w = *reinterpret_cast<const float4*>(weight + 4 * g);
        st_store4<TO>(o + 4 * g, make_float4(v[i].x * inv * w.x, v[i].y * inv * w.y, v[i].z * inv * w.z, v[i].w * inv * w.w));
      }
    }
  } else {
    auto value = [&](int c) {
      float s = 0.f;
      if (a) s = st_load1(a, a_dtype, base + c);
      if (b) s += st_load1(b, b_dtype, base + c);
      s *= m;
      if (first) s += first[base + c];
      if (vec) s += vec[c];
      return residual[base + c] + s;
    };
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float x = value(c);
      ss += x * x;
    }
    if (weight) {
      ss = ms_block_sum(ss, scratch);
      const float inv = rsqrtf(ss / (float)d + eps);
      TO* o = out + (size_t)orow * d;
      for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = ms_from_float<TO>(value(c) * inv * weight[c]);
    }
    if (adds && !rows) {
      __syncthreads();  // every thread has read what it needs of the old row
      for (int c = threadIdx.x; c < d; c += blockDim.x) residual[base + c] = value(c);
    }
  }
}

MS_API int ms_add_streams_rmsnorm(float* residual, const void* a, int a_dtype, const void* b, int b_dtype, const float* first,
                                  const float* vec, const float* weight, void* out, int out_dtype, const int* rows, int n_out, int d,
                                  float eps, float delta_scale, cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(n_out > 0 && d > 0, "add_streams_rmsnorm: bad sizes n_out=%d d=%d", n_out, d);
  MS_REQUIRE((a_dtype == MS_F32 || a_dtype == MS_BF16) && (b_dtype == MS_F32 || b_dtype == MS_BF16), "add_streams_rmsnorm: bad delta dtype");
  MS_REQUIRE(weight == nullptr || out != nullptr, "add_streams_rmsnorm: a weight without an output");
  const uintptr_t all = (uintptr_t)residual | (uintptr_t)a | (uintptr_t)b | (uintptr_t)first | (uintptr_t)vec | (uintptr_t)weight | (uintptr_t)out;
  const bool vecs = d % 4 == 0 && d <= 4 * ST_THREADS * ST_KEEP && all % 16 == 0;
#define MS_ST_LAUNCH(TO, V)                                                                                                       \
  MS_LAUNCH_RESULT("add_streams_rmsnorm", ms_launch(add_streams_rmsnorm_kernel<TO, V>, dim3(n_out), dim3(ST_THREADS), 0, stream, 1, \
                                                    true, residual, a, a_dtype, b, b_dtype, first, vec, weight, (TO*)out, rows, d, eps,     \
                                                    delta_scale))
  if (out_dtype == MS_BF16) {
    if (vecs) MS_ST_LAUNCH(__nv_bfloat16, true);
    else MS_ST_LAUNCH(__nv_bfloat16, false);
  } else if (out_dtype == MS_F32) {
    if (vecs) MS_ST_LAUNCH(float, true);
    else MS_ST_LAUNCH(float, false);
  } else {
    MS_REQUIRE(false, "add_streams_rmsnorm: unknown out dtype %d", out_dtype);
  }
#undef MS_ST_LAUNCH
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------

// One block a row; a and b float32 [rows, d]; the row's two sums of squares are taken side by side.  VEC: d is a multiple of
// 4, every pointer 16-byte aligned and d <= ST_THREADS * NP_KEEP * 4: both rows stay in registers between the two passes.
#define NP_KEEP 4
template <bool VEC>
__global__ void __launch_bounds__(ST_THREADS)
norm_pair_mean_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa, const float* __restrict__ wb,
                      float* __restrict__ out, int d, float eps, float m) {
  __shared__ float scratch_a[33], scratch_b[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t base = (size_t)blockIdx.x * d;
  float sa = 0.f, sb = 0.f;
  if constexpr (VEC) {
    float4 x[NP_KEEP], y[NP_KEEP];
    const int ngroups = d / 4;
    const float4* a4 = reinterpret_cast<const float4*>(a + base);
    const float4* b4 = reinterpret_cast<const float4*>(b + base);
#pragma unroll
    for (int i = 0; i < NP_KEEP; ++i) {
      const int g = threadIdx.x + i * ST_THREADS;
      if (g < ngroups) {
        x[i] = a4[g];
        y[i] = b4[g];
        sa += x[i].x * x[i].x + x[i].y * x[i].y + x[i].z * x[i].z + x[i].w * x[i].w;
        sb += y[i].x * y[i].x + y[i].y * y[i].y + y[i].z * y[i].z + y[i].w * y[i].w;
      }
    }
    sa = ms_block_sum(sa, scratch_a);
    sb = ms_block_sum(sb, scratch_b);
    const float ia = rsqrtf(sa / (float)d + eps), ib = rsqrtf(sb / (float)d + eps);
    float4* o4 = reinterpret_cast<float4*>(out + base);
#pragma unroll
    for (int i = 0; i < NP_KEEP; ++i) {
      const int g = threadIdx.x + i * ST_THREADS;
      if (g < ngroups) {
        const float4 p = reinterpret_cast<const float4*>(wa)[g], q = reinterpret_cast<const float4*>(wb)[g];
        float4 r;
        r.x = m * (x[i].x * ia * p.x + y[i].x * ib * q.x);
        r.y = m * (x[i].y * ia * p.y + y[i].y * ib * q.y);
        r.z = m * (x[i].z * ia * p.z + y[i].z * ib * q.z);
        r.w = m * (x[i].w * ia * p.w + y[i].w * ib * q.w);
        o4[g] = r;
      }
    }
  } else {
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float x = a[base + c], y = b[base + c];
      sa += x * x;
      sb += y * y;
    }
    sa = ms_block_sum(sa, scratch_a);
    sb = ms_block_sum(sb, scratch_b);
    const float ia = rsqrtf(sa / (float)d + eps), ib = rsqrtf(sb / (float)d + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[base + c] = m * (a[base + c] * ia * wa[c] + b[base + c] * ib * wb[c]);
  }
}

MS_API int ms_norm_pair_mean(const float* a, const float* b, const float* wa, const float* wb, float* out, int rows, int d, float eps,
                             float m, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && d > 0, "norm_pair_mean: bad sizes rows=%d d=%d", rows, d);
  const bool vec = d % 4 == 0 && d <= ST_THREADS * NP_KEEP * 4 &&
                   (((uintptr_t)a | (uintptr_t)b | (uintptr_t)wa | (uintptr_t)wb | (uintptr_t)out) & 15) == 0;
  if (vec)
    MS_LAUNCH_RESULT("norm_pair_mean", ms_launch(norm_pair_mean_kernel<true>, dim3(rows), dim3(ST_THREADS), 0, stream, 1, true, a, b, wa, wb,
                                                 out, d, eps, m));
  else
    MS_LAUNCH_RESULT("norm_pair_mean", ms_launch(norm_pair_mean_kernel<false>, dim3(rows), dim3(ST_THREADS), 0, stream, 1, true, a, b, wa, wb,
                                                 out, d, eps, m));
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------

template <bool VEC>
__global__ void __launch_bounds__(256)
pair_weighted_sum_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ bias_a,
                         const float* __restrict__ bias_b, float* __restrict__ out, int d, size_t total, float sa, float sb) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
  if (i >= total) return;
  if constexpr (VEC) {
    const int c = (int)(i % d);  // (d is a multiple of 4: the four lie in one row)
    float4 x = *reinterpret_cast<const float4*>(a + i), y = *reinterpret_cast<const float4*>(b + i);
    if (bias_a) {
      const float4 u = *reinterpret_cast<const float4*>(bias_a + c);
      x.x += u.x, x.y += u.y, x.z += u.z, x.w += u.w;
    }
    if (bias_b) {
      const float4 u = *reinterpret_cast<const float4*>(bias_b + c);
      y.x += u.x, y.y += u.y, y.z += u.z, y.w += u.w;
    }
    *reinterpret_cast<float4*>(out + i) = make_float4(sa * x.x + sb * y.x, sa * x.y + sb * y.y, sa * x.z + sb * y.z, sa * x.w + sb * y.w);
  } else {
    const int c = (int)(i % d);
    out[i] = sa * (a[i] + (bias_a ? bias_a[c] : 0.f)) + sb * (b[i] + (bias_b ? bias_b[c] : 0.f));
  }
}

MS_API int ms_pair_weighted_sum(const float* a, const float* b, const float* bias_a, const float* bias_b, float* out, int rows, int d,
                                float sa, float sb, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && d > 0, "pair_weighted_sum: bad sizes rows=%d d=%d", rows, d);
  const size_t total = (size_t)rows * d;
  const bool vec = d % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)bias_a | (uintptr_t)bias_b | (uintptr_t)out) & 15) == 0;
  const size_t threads = vec ? total / 4 : total;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (vec)
    MS_LAUNCH_RESULT("pair_weighted_sum", ms_launch(pair_weighted_sum_kernel<true>, dim3(blocks), dim3(256), 0, stream, 1, true, a, b, bias_a,
                                                    bias_b, out, d, total, sa, sb));
  else
    MS_LAUNCH_RESULT("pair_weighted_sum", ms_launch(pair_weighted_sum_kernel<false>, dim3(blocks), dim3(256), 0, stream, 1, true, a, b, bias_a,
                                                    bias_b, out, d, total, sa, sb));
  return 0;
}

// ------------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float st_act(float g, int act) {
  if (act == 0) return g / (1.f + expf(-g));
  if (act == 2) return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));  // the exact GELU
  // 0.5 g (1 + tanh(u)) = g / (1 + exp(-2u)): one accurate exponential and one division
  const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return g / (1.f + expf(-2.f * u));
}

// Four columns a thread with 16-byte (float32) or 8-byte (bfloat16) accesses, for widths that are a multiple of 4.
template <typename TI, typename TO>
__global__ void gated_act_mul_vec_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inter, int act) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= inter) return;
  const int dt = sizeof(TI) == 4 ? MS_F32 : MS_BF16;
  const float4 g = st_load4(gate_up, dt, (size_t)row * 2 * inter + c), u = st_load4(gate_up, dt, (size_t)row * 2 * inter + inter + c);
  st_store4<TO>(out + (size_t)row * inter + c, make_float4(st_act(g.x, act) * u.x, st_act(g.y, act) * u.y, st_act(g.z, act) * u.z,
                                                            st_act(g.w, act) * u.w));
}

template <typename TI, typename TO>
__global__ void gated_act_mul_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inter, int act) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= inter) return;
  const TI* p = gate_up + (size_t)row * 2 * inter;
  out[(size_t)row * inter + c] = ms_from_float<TO>(st_act(ms_to_float(p[c]), act) * ms_to_float(p[inter + c]));
}

// act: 0 SiLU, 1 GELU (tanh form), 2 GELU (exact).  gate_up [rows, 2*inter] float32 or bfloat16, out [rows, inter] float32 or bfloat16.
// Eight columns a thread with 16-byte accesses: bfloat16 in and out, widths that are a multiple of 8.
__global__ void gated_act_mul_vec8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter, int act) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= inter) return;
  const uint4 g = *reinterpret_cast<const uint4*>(gate_up + (size_t)row * 2 * inter + c);
  const uint4 u = *reinterpret_cast<const uint4*>(gate_up + (size_t)row * 2 * inter + inter + c);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 r;
  __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 gf = __bfloat1622float2(gh[i]), uf = __bfloat1622float2(uh[i]);
    rh[i] = __floats2bfloat162_rn(st_act(gf.x, act) * uf.x, st_act(gf.y, act) * uf.y);
  }
  *reinterpret_cast<uint4*>(out + (size_t)row * inter + c) = r;
}

MS_API int ms_gated_act_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int rows, int inter, int act, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && rows <= 65535 * 64 && inter > 0 && act >= 0 && act <= 2, "gated_act_mul: bad arguments rows=%d inter=%d act=%d", rows,
             inter, act);
  MS_REQUIRE(rows <= 65535, "gated_act_mul: %d rows are more than one launch takes", rows);
  if (in_dtype == MS_BF16 && out_dtype == MS_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up | (uintptr_t)out) % 16 == 0) {
    MS_LAUNCH_RESULT("gated_act_mul", ms_launch(gated_act_mul_vec8_kernel, dim3((inter / 8 + 127) / 128, rows), dim3(128), 0, stream, 1, true,
                                                (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, act));
    return 0;
  }
  const bool vec = inter % 4 == 0 && ((uintptr_t)gate_up | (uintptr_t)out) % 16 == 0;
  const dim3 grid(vec ? (inter / 4 + 127) / 128 : (inter + 255) / 256, rows);
#define MS_GA_LAUNCH(TI, TO)                                                                                                          \
  do {                                                                                                                                \
    if (vec)                                                                                                                          \
      MS_LAUNCH_RESULT("gated_act_mul", ms_launch(gated_act_mul_vec_kernel<TI, TO>, grid, dim3(128), 0, stream, 1, true,              \
                                                  (const TI*)gate_up, (TO*)out, inter, act));                                         \
    else                                                                                                                              \
      MS_LAUNCH_RESULT("gated_act_mul", ms_launch(gated_act_mul_kernel<TI, TO>, grid, dim3(256), 0, stream, 1, true,                  \
                                                  (const TI*)gate_up, (TO*)out, inter, act));                                         \
  } while (0)
  if (in_dtype == MS_F32 && out_dtype == MS_F32) MS_GA_LAUNCH(float, float);
  else if (in_dtype == MS_F32 && out_dtype == MS_BF16) MS_GA_LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == MS_BF16 && out_dtype == MS_BF16) MS_GA_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == MS_BF16 && out_dtype == MS_F32) MS_GA_LAUNCH(__nv_bfloat16, float);
  else MS_REQUIRE(false, "gated_act_mul: unknown dtypes %d -> %d", in_dtype, out_dtype);
#undef MS_GA_LAUNCH
  return 0;
}
