// Rotation of queries and keys by position and the write of keys and values into their pages, for a mixer whose keys and
// values have widths of their own: what stands between the q|k|v product and the attention.
//
// For every row t of proj [T, ld] = [q (Hq*dk) | k (G*dk) | v (G*dv)], float32 (plus `bias`, float32 over the same columns,
// where one is given: the projections' biases are added as the product is read), at position p:
//   the first `rot` coordinates of every query and key head are turned in pairs by the angles of the table
//   cos_sin [positions, rot/2, 2] (cos, sin of p * f_i, made on the host in float64): pair i is (i, i + rot/2) ("half") or
//   (2i, 2i + 1) (interleaved); (a, b) becomes (a cos - b sin, b cos + a sin).  The other coordinates pass unchanged.
// The queries go to q_out [T, Hq*dk] in float32 (and, rounded, to q_half if that is given); the keys and the values go
// to the pages of the row's request at its position, in the cache's type: k pages [pages, G, page, dk], v pages
// [pages, G, page, dv].  Rows without a request (slot < 0) are passed over.  All arithmetic is float32.
#include "launch.cuh"

__device__ __forceinline__ float rs_turned(const float* head, const float* bias, int e, int rot, int interleaved, const float* cs) {
  if (e >= rot) return bias ? head[e] + bias[e] : head[e];
  const int half = rot >> 1;
  int i, first;
  float a, b;
  if (interleaved) {
    i = e >> 1;
    first = !(e & 1);
    a = head[2 * i];
    b = head[2 * i + 1];
    if (bias) {
      a += bias[2 * i];
      b += bias[2 * i + 1];
    }
  } else {
    first = e < half;
    i = first ? e : e - half;
    a = head[i];
    b = head[i + half];
    if (bias) {
      a += bias[i];
      b += bias[i + half];
    }
  }
  const float c = cs[2 * i], s = cs[2 * i + 1];
  return first ? a * c - b * s : b * c + a * s;
}

template <typename TC>
__global__ void __launch_bounds__(256)
rope_store_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias, const float* __restrict__ cos_sin, int rot, int interleaved, int max_pos,
                  const int* __restrict__ positions, const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                  int num_pages, int page_size, float* __restrict__ q_out, __nv_bfloat16* __restrict__ q_half, TC* __restrict__ k_pages,
                  TC* __restrict__ v_pages, int heads, int groups, int dk, int dv, int store) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int pos = positions[t];
  const float* row = proj + (size_t)t * ld;
  const float* cs = cos_sin + (size_t)(pos < max_pos ? pos : max_pos - 1) * rot;  // (positions are checked on the host)
  const int qw = heads * dk, kw = groups * dk, vw = groups * dv;
  for (int c = threadIdx.x; c < qw; c += blockDim.x) {
    const int h = c / dk, e = c - h * dk;
    const float o = rs_turned(row + h * dk, bias ? bias + h * dk : nullptr, e, rot, interleaved, cs);
    q_out[(size_t)t * qw + c] = o;
    if (q_half) q_half[(size_t)t * qw + c] = __float2bfloat16_rn(o);
  }
  if (!store) return;
  const int page = block_table[(size_t)slot * max_pages + pos / page_size];
  if (page < 0 || page >= num_pages) return;
  const size_t at = (size_t)page * groups * page_size + pos % page_size;  // + g * page_size: the row of the (page, head) arrays
  for (int c = threadIdx.x; c < kw; c += blockDim.x) {
    const int g = c / dk, e = c - g * dk;
    k_pages[(at + (size_t)g * page_size) * dk + e] = ms_from_float<TC>(rs_turned(row + qw + g * dk, bias ? bias + qw + g * dk : nullptr, e, rot, interleaved, cs));
  }
  for (int c = threadIdx.x; c < vw; c += blockDim.x) {
    const int g = c / dv, e = c - g * dv;
    v_pages[(at + (size_t)g * page_size) * dv + e] = ms_from_float<TC>(bias ? row[qw + kw + c] + bias[qw + kw + c] : row[qw + kw + c]);
  }
}

MS_API int ms_rope_store(const float* proj, int ld, const float* bias, const float* cos_sin, int rot, int interleaved, int max_pos, const int* positions,
                         const int* slots, const int* block_table, int max_pages, int num_pages, int page_size, float* q_out, void* q_half,
                         void* k_pages, void* v_pages, int cache_dtype, int tokens, int heads, int groups, int dk, int dv, int store,
                         cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && heads > 0 && groups > 0 && dk > 0 && dv > 0, "rope_store: bad sizes");
  MS_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk && (rot == 0 || (cos_sin != nullptr && max_pos > 0)), "rope_store: %d of %d coordinates cannot be rotated", rot, dk);
  MS_REQUIRE(ld >= heads * dk + (store ? groups * (dk + dv) : 0), "rope_store: rows of %d elements do not hold q, k and v", ld);
  MS_REQUIRE(!store || (max_pages > 0 && num_pages > 0 && page_size > 0 && k_pages && v_pages), "rope_store: no cache to write");
  if (cache_dtype == MS_F32)
    MS_LAUNCH_RESULT("rope_store", ms_launch(rope_store_kernel<float>, dim3(tokens), dim3(256), 0, stream, 1, true, proj, ld, bias, cos_sin, rot,
                                             interleaved, max_pos, positions, slots, block_table, max_pages, num_pages, page_size, q_out,
                                             (__nv_bfloat16*)q_half, (float*)k_pages, (float*)v_pages, heads, groups, dk, dv, store));
  else if (cache_dtype == MS_BF16)
    MS_LAUNCH_RESULT("rope_store", ms_launch(rope_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, 1, true, proj, ld, bias, cos_sin,
                                             rot, interleaved, max_pos, positions, slots, block_table, max_pages, num_pages, page_size,
                                             q_out, (__nv_bfloat16*)q_half, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, heads, groups, dk,
                                             dv, store));
  else
    MS_REQUIRE(false, "rope_store: unknown cache dtype %d", cache_dtype);
  return 0;
}
