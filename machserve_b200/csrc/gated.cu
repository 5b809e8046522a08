// Gated activations beside SiLU-mul: the clamped gated unit of a feed-forward, and a sigmoid gate on a mixer's output.
//
// clamped gated unit: gate_up is float32 [rows, 2*inter] (gate in columns [0, inter), up in [inter, 2*inter)), out the type
// the next product reads;
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + shift).
// sigmoid gate: out[r, c] = x[r, c] * sigmoid(gate[r, c]); x and gate are float32 with row strides of their own
//   (a gate that is a column range of a wider product), out is the type the next product reads.
// Both compute in float32 with the accurate expf.
#include "launch.cuh"

template <typename T>
__global__ void glu_clamped_kernel(const float* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total, float limit,
                                   float alpha, float shift) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / inter;
  const int c = (int)(i - r * inter);
  const float g = fminf(gate_up[r * 2 * inter + c], limit);
  const float u = fminf(fmaxf(gate_up[r * 2 * inter + inter + c], -limit), limit);
  out[i] = ms_from_float<T>(g / (1.f + expf(-alpha * g)) * (u + shift));
}

// Eight columns per thread with 16- and 32-byte accesses, for widths that are a multiple of 8.
template <typename T>
__global__ void glu_clamped_vec_kernel(const float* __restrict__ gate_up, T* __restrict__ out, int inter, float limit, float alpha,
                                       float shift) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= inter) return;
  const float* gp = gate_up + (size_t)row * 2 * inter + c;
  const float4 g0 = *reinterpret_cast<const float4*>(gp), g1 = *reinterpret_cast<const float4*>(gp + 4);
  const float4 u0 = *reinterpret_cast<const float4*>(gp + inter), u1 = *reinterpret_cast<const float4*>(gp + inter + 4);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  float r[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float gk = fminf(g[k], limit), uk = fminf(fmaxf(u[k], -limit), limit);
    r[k] = gk / (1.f + expf(-alpha * gk)) * (uk + shift);
  }
  T* o = out + (size_t)row * inter + c;
  if constexpr (sizeof(T) == 2) {
    uint4 pk;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(r[2 * k], r[2 * k + 1]);
    *reinterpret_cast<uint4*>(o) = pk;
  } else {
    *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(o + 4) = make_float4(r[4], r[5], r[6], r[7]);
  }
}

MS_API int ms_glu_clamped(const float* gate_up, void* out, int dtype, int rows, int inter, float limit, float alpha, float shift,
                          cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && inter > 0 && limit > 0.f, "glu_clamped: bad arguments rows=%d inter=%d limit=%g", rows, inter, limit);
  if (inter % 8 == 0 && rows <= 65535 && ((uintptr_t)gate_up | (uintptr_t)out) % 16 == 0 && (dtype == MS_F32 || dtype == MS_BF16)) {
    dim3 grid((inter / 8 + 127) / 128, rows);
    if (dtype == MS_F32)
      MS_LAUNCH_RESULT("glu_clamped", ms_launch(glu_clamped_vec_kernel<float>, grid, dim3(128), 0, stream, 1, true, gate_up, (float*)out,
                                                inter, limit, alpha, shift));
    else
      MS_LAUNCH_RESULT("glu_clamped", ms_launch(glu_clamped_vec_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, true, gate_up,
                                                (__nv_bfloat16*)out, inter, limit, alpha, shift));
    return 0;
  }
  const size_t total = (size_t)rows * inter;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH_RESULT("glu_clamped", ms_launch(glu_clamped_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true,
                                              gate_up, (float*)out, inter, total, limit, alpha, shift));
  else if (dtype == MS_BF16)
    MS_LAUNCH_RESULT("glu_clamped", ms_launch(glu_clamped_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true,
                                              gate_up, (__nv_bfloat16*)out, inter, total, limit, alpha, shift));
  else
    MS_REQUIRE(false, "glu_clamped: unknown dtype %d", dtype);
  return 0;
}

template <typename TO>
__global__ void sigmoid_gate_mul_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gate, int ldg,
                                        TO* __restrict__ out, int n, size_t total) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / n;
  const int c = (int)(i - r * n);
  const float g = gate[r * ldg + c];
  out[i] = ms_from_float<TO>(x[r * ldx + c] / (1.f + expf(-g)));
}

MS_API int ms_sigmoid_gate_mul(const float* x, int ldx, const float* gate, int ldg, void* out, int out_dtype, int rows, int n,
                               cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && n > 0 && ldx >= n && ldg >= n, "sigmoid_gate_mul: bad sizes rows=%d n=%d", rows, n);
  const size_t total = (size_t)rows * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("sigmoid_gate_mul", ms_launch(sigmoid_gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true, x, ldx,
                                                   gate, ldg, (float*)out, n, total));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("sigmoid_gate_mul", ms_launch(sigmoid_gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true,
                                                   x, ldx, gate, ldg, (__nv_bfloat16*)out, n, total));
  else
    MS_REQUIRE(false, "sigmoid_gate_mul: unknown out dtype %d", out_dtype);
  return 0;
}

// A sigmoid gate per head on a mixer's output: out[r, h*dv + c] = x[r, h*dv + c] * sigmoid(gate[r, h]).  x and out are of
// one type (the type the next product reads) and may be the same array; gate is float32 with a row stride of its own (a
// column range of a wider product).  The product is float32.
template <typename T>
__global__ void head_gate_mul_kernel(const T* x, const float* __restrict__ gate, int ldg, T* out, int heads, int dv, size_t total) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int n = heads * dv;
  const size_t r = i / n;
  const int h = (int)(i - r * n) / dv;
  const float g = gate[r * ldg + h];
  out[i] = ms_from_float<T>(ms_to_float(x[i]) * (1.f / (1.f + expf(-g))));
}

// The same with 16 bytes a thread (dv a multiple of the 16 / sizeof(T) elements that a thread takes, so that they lie in
// one head; x and out 16-byte aligned): an element's arithmetic is that of the kernel above.
#define HG_ROWS 4  // rows a thread takes: their loads are all requested before the first is used
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_mul_vec_kernel(const T* x, const float* __restrict__ gate, int ldg, T* out, int rows, int dv, int per_row) {
  constexpr int E = 16 / sizeof(T);
  ms_pdl_trigger();
  ms_pdl_wait();
  const int j = blockIdx.x * blockDim.x + threadIdx.x;  // (threads are laid out by rows: no division finds the row)
  if (j >= per_row) return;
  const size_t r0 = (size_t)blockIdx.y * (blockDim.y * HG_ROWS) + threadIdx.y;
  union V {
    uint4 u;
    T e[E];
  };
  uint4 raw[HG_ROWS];
  float g[HG_ROWS];
#pragma unroll
  for (int k = 0; k < HG_ROWS; ++k) {
    const size_t r = r0 + (size_t)k * blockDim.y;
    if (r < (size_t)rows) {
      raw[k] = (reinterpret_cast<const uint4*>(x) + r * per_row)[j];
      g[k] = gate[r * ldg + j * E / dv];
    }
  }
#pragma unroll
  for (int k = 0; k < HG_ROWS; ++k) {
    const size_t r = r0 + (size_t)k * blockDim.y;
    if (r < (size_t)rows) {
      const float s = 1.f / (1.f + expf(-g[k]));  // one division a head and thread, a product an element
      V v;
      v.u = raw[k];
#pragma unroll
      for (int i = 0; i < E; ++i) v.e[i] = ms_from_float<T>(ms_to_float(v.e[i]) * s);
      (reinterpret_cast<uint4*>(out) + r * per_row)[j] = v.u;
    }
  }
}

MS_API int ms_head_gate_mul(const void* x, const float* gate, int ldg, void* out, int dtype, int rows, int heads, int dv,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && heads > 0 && dv > 0 && ldg >= heads, "head_gate_mul: bad sizes rows=%d heads=%d dv=%d", rows, heads, dv);
  const size_t total = (size_t)rows * heads * dv;
  const int per = dtype == MS_F32 ? 4 : 8;
  if ((dtype == MS_F32 || dtype == MS_BF16) && dv % per == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0 && rows <= 65535) {
    const int per_row = heads * dv / per;
    int tx = 32;
    while (tx < 256 && tx < per_row) tx *= 2;
    const int per_block = 256 / tx * HG_ROWS;
    const dim3 threads(tx, 256 / tx), grid((per_row + tx - 1) / tx, (rows + per_block - 1) / per_block);
    if (dtype == MS_F32)
      MS_LAUNCH_RESULT("head_gate_mul", ms_launch(head_gate_mul_vec_kernel<float>, grid, threads, 0, stream, 1, true, (const float*)x, gate,
                                                  ldg, (float*)out, rows, dv, per_row));
    else
      MS_LAUNCH_RESULT("head_gate_mul", ms_launch(head_gate_mul_vec_kernel<__nv_bfloat16>, grid, threads, 0, stream, 1, true,
                                                  (const __nv_bfloat16*)x, gate, ldg, (__nv_bfloat16*)out, rows, dv, per_row));
    return 0;
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH_RESULT("head_gate_mul", ms_launch(head_gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, true, (const float*)x, gate,
                                                ldg, (float*)out, heads, dv, total));
  else if (dtype == MS_BF16)
    MS_LAUNCH_RESULT("head_gate_mul", ms_launch(head_gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, 1, true,
                                                (const __nv_bfloat16*)x, gate, ldg, (__nv_bfloat16*)out, heads, dv, total));
  else
    MS_REQUIRE(false, "head_gate_mul: unknown dtype %d", dtype);
  return 0;
}
