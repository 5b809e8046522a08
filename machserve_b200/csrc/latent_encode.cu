// What stands between the input product of a latent-attention mixer and its attention: the norm of the latent, the
// rotation of the shared key part and of the queries' rotated parts, and the write of [latent | rotated key part]
// into the one plane of pages that the mixer keeps.
//
// Row t of proj [T, ld], float32, holds the queries at column 0, head by head as [dn unrotated | dr rotated], and
// at column kv_off the down-projection [r latent | dr key part].
//   c  = latent / sqrt(mean(latent^2) + eps) * w            -> pages[.., 0:r]
//   kr = turn(key part, p)                                   -> pages[.., r:r+dr]
//   q_wide[t, h, r:r+dr] = turn(q[t, h, dn:dn+dr], p)        (float32; columns 0:r are filled by the product of the
//                                                             unrotated queries with the keys' up-projection)
//   q_plain[t, h, :] = q[t, h, 0:dn]                          (in the type that product reads)
// turn: the pair (2i, 2i+1) (interleaved) or (i, i + rot/2) (halves), i < rot/2, at position p becomes
// (u cos a - v sin a, v cos a + u sin a) with (cos a, sin a) from the table [positions, rot/2, 2]; coordinates from `rot`
// on pass unchanged.  The queries may come from a product of their own (`q_src` [T, q_ld], head by head from column 0:
// a mixer whose queries pass a latent too) instead of from column 0 of proj.  Rows without a request (slot < 0)
// are passed over.  float32 arithmetic throughout.
#include "launch.cuh"

__device__ __forceinline__ float latent_turn(const float* x, int e, int rot, int interleaved, const float* cs) {
  if (e >= rot) return x[e];
  const int half = rot >> 1;
  const bool second = interleaved ? (e & 1) : e >= half;
  const int i = interleaved ? e >> 1 : (second ? e - half : e);
  const float c = cs[2 * i], s = cs[2 * i + 1];
  const float u = interleaved ? x[2 * i] : x[i], v = interleaved ? x[2 * i + 1] : x[i + half];
  return second ? v * c + u * s : u * c - v * s;
}

// Four coordinates e..e+3 (e a multiple of 4) of a vector whose first `rot` (a multiple of 8) are turned in halves.
__device__ __forceinline__ float4 latent_turn4_halves(const float* x, int e, int rot, const float* cs) {
  const float4 a = *reinterpret_cast<const float4*>(x + e);
  if (e >= rot) return a;
  const int half = rot >> 1;
  const bool second = e >= half;
  const int i = second ? e - half : e;
  const float4 b = *reinterpret_cast<const float4*>(x + (second ? i : e + half));  // the partners
  const float4 c0 = *reinterpret_cast<const float4*>(cs + 2 * i), c1 = *reinterpret_cast<const float4*>(cs + 2 * i + 4);
  // (cos, sin) of pairs i, i+1 in c0 and i+2, i+3 in c1; first half: u c - v s with u = a, v = b; second half: v c + u s with v = a, u = b
  const float sg = second ? 1.f : -1.f;
  return make_float4(a.x * c0.x + sg * b.x * c0.y, a.y * c0.z + sg * b.y * c0.w, a.z * c1.x + sg * b.z * c1.y, a.w * c1.z + sg * b.w * c1.w);
}
__device__ __forceinline__ void latent_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void latent_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&lo);
  u.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TC, typename TN>
__global__ void __launch_bounds__(256)
latent_encode_kernel(const float* __restrict__ proj, int ld, int kv_off, const float* __restrict__ q_src, int q_ld,
                     const float* __restrict__ w_latent, float eps,
                     const float* __restrict__ cos_sin, int rot, int interleaved, const int* __restrict__ positions,
                     const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages, int num_pages,
                     int page_size, float* __restrict__ q_wide, TN* __restrict__ q_plain, TC* __restrict__ pages, int heads,
                     int dn, int dr, int r, int store, int vec) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int pos = positions[t];
  const float* row = proj + (size_t)t * ld;
  const float* qrow = q_src ? q_src + (size_t)t * q_ld : row;
  const float* cs = cos_sin + (size_t)pos * rot;  // [rot/2][2]
  const int hd = dn + dr, wide = r + dr;
  if (vec) {  // every size a multiple of 4, rotation in halves of a multiple of 8, rows on 16-byte boundaries: four elements a thread
    for (int c = threadIdx.x * 4; c < heads * hd; c += blockDim.x * 4) {
      const int h = c / hd, e = c - h * hd;
      if (e < dn)
        latent_store4(q_plain + ((size_t)t * heads + h) * dn + e, *reinterpret_cast<const float4*>(qrow + c));
      else
        latent_store4(q_wide + ((size_t)t * heads + h) * wide + r + (e - dn), latent_turn4_halves(qrow + h * hd + dn, e - dn, rot, cs));
    }
    if (!store) return;
    const float* kv = row + kv_off;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < r; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(kv + c);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float inv = 1.f / sqrtf(ms_block_sum(ss, scratch) / (float)r + eps);
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) return;
    TC* dst = pages + ((size_t)page * page_size + pos % page_size) * wide;
    for (int c = threadIdx.x * 4; c < wide; c += blockDim.x * 4) {
      float4 v;
      if (c < r) {
        const float4 x = *reinterpret_cast<const float4*>(kv + c), w = *reinterpret_cast<const float4*>(w_latent + c);
        v = make_float4(x.x * inv * w.x, x.y * inv * w.y, x.z * inv * w.z, x.w * inv * w.w);
      } else {
        v = latent_turn4_halves(kv + r, c - r, rot, cs);
      }
      latent_store4(dst + c, v);
    }
    return;
  }
  for (int c = threadIdx.x; c < heads * hd; c += blockDim.x) {
    const int h = c / hd, e = c - h * hd;
    if (e < dn)
      q_plain[((size_t)t * heads + h) * dn + e] = ms_from_float<TN>(qrow[c]);
    else
      q_wide[((size_t)t * heads + h) * wide + r + (e - dn)] = latent_turn(qrow + h * hd + dn, e - dn, rot, interleaved, cs);
  }
  if (!store) return;
  const float* kv = row + kv_off;
  float ss = 0.f;
  for (int c = threadIdx.x; c < r; c += blockDim.x) ss += kv[c] * kv[c];
  const float inv = 1.f / sqrtf(ms_block_sum(ss, scratch) / (float)r + eps);
  const int page = block_table[(size_t)slot * max_pages + pos / page_size];
  if (page < 0 || page >= num_pages) return;
  TC* dst = pages + ((size_t)page * page_size + pos % page_size) * wide;
  for (int c = threadIdx.x; c < wide; c += blockDim.x)
    dst[c] = ms_from_float<TC>(c < r ? kv[c] * inv * w_latent[c] : latent_turn(kv + r, c - r, rot, interleaved, cs));
}

MS_API int ms_latent_encode(const float* proj, int ld, int kv_off, const float* q_src, int q_ld, const float* w_latent, float eps,
                            const float* cos_sin, int rot, int interleaved, int table_positions, const int* positions, const int* slots, const int* block_table,
                            int max_pages, int num_pages, int page_size, float* q_wide, void* q_plain, int plain_dtype,
                            void* pages, int cache_dtype, int tokens, int heads, int dn, int dr, int r, int store,
                            cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && heads > 0 && dn > 0 && dr >= 0 && r > 0, "latent_encode: bad sizes");
  MS_REQUIRE(rot >= 0 && rot <= dr && rot % 2 == 0, "latent_encode: %d rotated coordinates of %d", rot, dr);
  MS_REQUIRE(rot == 0 || (cos_sin && table_positions > 0), "latent_encode: no table of angles");
  MS_REQUIRE((q_src ? q_ld : ld) >= heads * (dn + dr) && ld >= kv_off + (store ? r + dr : 0),
             "latent_encode: rows of %d elements are too short", ld);
  const bool halves_ok = rot == 0 || (!interleaved && rot % 8 == 0);
  const int vec = halves_ok && dn % 4 == 0 && dr % 4 == 0 && r % 4 == 0 && ld % 4 == 0 && kv_off % 4 == 0 && (!q_src || q_ld % 4 == 0) &&
                  (((uintptr_t)proj | (uintptr_t)q_src | (uintptr_t)w_latent | (uintptr_t)cos_sin | (uintptr_t)q_wide | (uintptr_t)q_plain |
                    (uintptr_t)pages) & 15) == 0;
  MS_REQUIRE(!store || (max_pages > 0 && num_pages > 0 && page_size > 0 && pages), "latent_encode: no cache to write");
#define MS_LATENT(TC, TN)                                                                                                 \
  MS_LAUNCH_RESULT("latent_encode", ms_launch(latent_encode_kernel<TC, TN>, dim3(tokens), dim3(256), 0, stream, 1, true, proj, ld, \
                                              kv_off, q_src, q_ld, w_latent, eps, cos_sin, rot, interleaved, positions, slots, block_table, max_pages,      \
                                              num_pages, page_size, q_wide, (TN*)q_plain, (TC*)pages, heads, dn, dr, r, store, vec))
  if (cache_dtype == MS_F32 && plain_dtype == MS_F32)
    MS_LATENT(float, float);
  else if (cache_dtype == MS_BF16 && plain_dtype == MS_BF16)
    MS_LATENT(__nv_bfloat16, __nv_bfloat16);
  else if (cache_dtype == MS_BF16 && plain_dtype == MS_F32)
    MS_LATENT(__nv_bfloat16, float);
  else
    MS_REQUIRE(false, "latent_encode: unsupported dtypes cache=%d queries=%d", cache_dtype, plain_dtype);
#undef MS_LATENT
  return 0;
}
