// The arithmetic of head preparation for one head held by one warp, shared by the kernel that
// prepares heads on its own (head_prep.cu) and by decode attention, which prepares its heads
// itself (attention_decode.cu): both must round alike, since a key written to the cache by one
// is read next to keys written by the other.
//
// Layout: head size HD = 32 * VEC; lane l holds elements [l * VEC, l * VEC + VEC); the rotation
// partner of element i (i +- HD/2) lives in lane l ^ 16 at the same place.
//
// Per head (infer/forward.odin:60-86): optional RMSNorm over the head with a weight per
// element (ss = sum x^2; ss /= n; ss += eps; r = 1/sqrt(ss); x = w * (r * x), infer/ops.odin:7-19),
// then the rotation of the pairs (i, i + HD/2) by the position's angles (infer/ops.odin:40-60).
#pragma once

#include "common.cuh"

namespace headmath {

template <int VEC>
__device__ __forceinline__ void load_vec(const bf16* p, float (&v)[VEC]) {
    if (VEC == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x; v[1] = a.y; v[2 % VEC] = b.x; v[3 % VEC] = b.y;
    } else {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
        v[0] = a.x; v[1] = a.y;
    }
}
template <int VEC>
__device__ __forceinline__ void load_vec(const float* p, float (&v)[VEC]) {
    if (VEC == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2 % VEC] = a.z; v[3 % VEC] = a.w;
    } else {
        const float2 a = *reinterpret_cast<const float2*>(p);
        v[0] = a.x; v[1] = a.y;
    }
}
template <int VEC>
__device__ __forceinline__ void store_vec_bf16(bf16* p, const float (&o)[VEC]) {
    if (VEC == 4) {
        __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2 % VEC], o[3 % VEC]);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]);
        *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(&a);
    }
}

// One head's elements of this lane: the first part, then the other parts of a split product,
// four loads in flight at a time, added in their order.
template <int VEC, typename TI>
__device__ __forceinline__ void load_parts(const TI* src, int n_split, size_t split_stride, float (&v)[VEC]) {
    load_vec<VEC>(src, v);
    for (int s0 = 1; s0 < n_split; s0 += 4) {
        float w2[4][VEC];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (s0 + u < n_split) load_vec<VEC>(src + (size_t)(s0 + u) * split_stride, w2[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (s0 + u < n_split) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[e] += w2[u][e];
            }
    }
}

// v: this lane's elements of the head; wn: the norm's weights at the same places; c, sn: the
// cosines and sines of the position's angles at this lane's places of the first half.
template <int VEC>
__device__ __forceinline__ void norm_rotate(float (&v)[VEC], bool has_norm, const float (&wn)[VEC], float eps,
                                            bool rotate, const float (&c)[VEC], const float (&sn)[VEC], int lane,
                                            float (&o)[VEC]) {
    constexpr int HD = VEC * 32;
    if (has_norm) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += v[e] * v[e];
        ss = warp_sum(ss);
        ss /= (float)HD;
        ss += eps;
        const float r = 1.0f / sqrtf(ss);
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = wn[e] * (r * v[e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
        // first half: x c - y s with (x, y) = (mine, other); second half: x s + y c with (x, y) = (other, mine)
        if (rotate) o[e] = (lane < 16) ? (v[e] * c[e] - other * sn[e]) : (other * sn[e] + v[e] * c[e]);
        else o[e] = v[e];
    }
}

}  // namespace headmath
