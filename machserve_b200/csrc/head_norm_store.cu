// Between the q|k(|v) product of an attention mixer and its attention, for mixers that norm each head on its own:
//
//   q_h <- q_h / rms(q_h) (* wq),  k_g <- k_g / rms(k_g) (* wk)      rms over the head's dk coordinates, eps inside the root;
//   the normed keys go into the "k" pages; the values go into the "v" pages: a projection of their own (dv wide, at
//   v_off of the product), or, v_off < 0, the keys as they were projected, before their norm.
// proj is float32 [T, ld] = [q (hq*dk) | k (hkv*dk) | v], to which `bias` (float32, the same columns, or null) is added first;
// q_out float32 [T, hq*dk] and, optionally, a bfloat16 copy.
// With coef != 0 the normed query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
// One warp a head; the sums are float32 and their order depends on dk alone.  norm = 0 leaves q and k as they are.
#include "launch.cuh"

template <typename TC>
__global__ void __launch_bounds__(128)
head_norm_store_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias, const float* __restrict__ wq,
                       const float* __restrict__ wk, float eps, float coef, int every,
                       int norm, const int* __restrict__ positions, const int* __restrict__ slots, const int* __restrict__ block_table,
                       int max_pages, int num_pages, int page_size, float* __restrict__ q_out, __nv_bfloat16* __restrict__ q_half,
                       TC* __restrict__ k_pages, TC* __restrict__ v_pages, int hq, int hkv, int dk, int dv, int v_off, int store) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float* row = proj + (size_t)t * ld;
  const int slot = slots[t];
  int page = -1, off = 0;
  const float temp = (coef != 0.f && slot >= 0) ? 1.f + coef * logf((float)((positions[t] + 1) / every + 1)) : 1.f;
  if (store && slot >= 0) {
    const int p = positions[t];
    page = block_table[(size_t)slot * max_pages + p / page_size];
    off = p % page_size;
    if (page < 0 || page >= num_pages) page = -1;
  }
  const int nheads = store ? hq + hkv : hq;  // (a run that reads another run's cache projects the queries only)
  for (int h = warp; h < nheads; h += nwarps) {
    const bool is_q = h < hq;
    const float* xr = row + (size_t)h * dk;  // q heads, then k heads, lie side by side
    const float* br = bias ? bias + (size_t)h * dk : nullptr;
    auto x = [&](int d) { return br ? xr[d] + br[d] : xr[d]; };
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) ss += x(d) * x(d);
    ss = ms_warp_sum(ss);
    const float inv = norm ? rsqrtf(ss / (float)dk + eps) : 1.f;
    const float* w = is_q ? wq : wk;
    if (is_q) {
      for (int d = lane; d < dk; d += 32) {
        const float v = x(d) * inv * (w ? w[d] : 1.f) * temp;
        q_out[((size_t)t * hq + h) * dk + d] = v;
        if (q_half) q_half[((size_t)t * hq + h) * dk + d] = __float2bfloat16_rn(v);
      }
    } else if (page >= 0) {
      const int g = h - hq;
      const size_t cell = ((size_t)page * hkv + g) * page_size + off;
      for (int d = lane; d < dk; d += 32) k_pages[cell * dk + d] = ms_from_float<TC>(x(d) * inv * (w ? w[d] : 1.f));
      if (v_off < 0) {
        for (int d = lane; d < dk; d += 32) v_pages[cell * dv + d] = ms_from_float<TC>(x(d));
      } else {
        const float* v = row + v_off + (size_t)g * dv;
        const float* bv = bias ? bias + v_off + (size_t)g * dv : nullptr;
        for (int d = lane; d < dv; d += 32) v_pages[cell * dv + d] = ms_from_float<TC>(bv ? v[d] + bv[d] : v[d]);
      }
    }
  }
}

MS_API int ms_head_norm_store(const float* proj, int ld, const float* bias, const float* wq, const float* wk, float eps, float coef,
                              int every, int norm, const int* positions,
                              const int* slots, const int* block_table, int max_pages, int num_pages, int page_size, float* q_out,
                              void* q_half, void* k_pages, void* v_pages, int cache_dtype, int tokens, int hq, int hkv, int dk, int dv,
                              int v_off, int store, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv > 0 && dk > 0 && dv > 0 && (coef == 0.f || every > 0), "head_norm_store: bad sizes");
  MS_REQUIRE(v_off >= 0 || dv == dk, "head_norm_store: values that are the keys have the keys' width (%d, not %d)", dk, dv);
  MS_REQUIRE(ld >= (store ? hq + hkv : hq) * dk && (!store || v_off < 0 || ld >= v_off + hkv * dv),
             "head_norm_store: the product's rows are too short (%d)", ld);
  MS_REQUIRE(!store || (max_pages > 0 && num_pages > 0 && page_size > 0 && k_pages && v_pages), "head_norm_store: bad cache");
  if (cache_dtype == MS_F32)
    MS_LAUNCH_RESULT("head_norm_store", ms_launch(head_norm_store_kernel<float>, dim3(tokens), dim3(128), 0, stream, 1, true, proj, ld, bias,
                                                  wq, wk, eps, coef, every, norm, positions, slots, block_table, max_pages, num_pages, page_size, q_out,
                                                  (__nv_bfloat16*)q_half, (float*)k_pages, (float*)v_pages, hq, hkv, dk, dv, v_off, store));
  else if (cache_dtype == MS_BF16)
    MS_LAUNCH_RESULT("head_norm_store", ms_launch(head_norm_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, 1, true, proj,
                                                  ld, bias, wq, wk, eps, coef, every, norm, positions, slots, block_table, max_pages, num_pages, page_size,
                                                  q_out, (__nv_bfloat16*)q_half, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, hq, hkv,
                                                  dk, dv, v_off, store));
  else
    MS_REQUIRE(false, "head_norm_store: unknown cache dtype %d", cache_dtype);
  return 0;
}
