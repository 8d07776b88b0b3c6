// agb_device.cuh -- device-side building blocks shared by the sm_100a kernels:
// mbarrier + bulk-async-copy (TMA unit, untiled, no multicast) wrappers with bounded waits,
// 16-byte vector load/convert helpers, and the strictly-rounded fp32 arithmetic that keeps
// every rounding point of the reference's op-by-op composition.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace agb {

// Device-global status word: 0 = ok, otherwise an agb_status_t written by a kernel whose
// bounded wait ran out.  Read and cleared by agb_device_status().
// (defined here: the library is a single translation unit)
__device__ int g_device_status = 0;

// A wait gives up after kWaitPollLimit polls of mbarrier.try_wait, each of which may suspend the
// thread in hardware for up to kWaitSuspendNs: at most ~2.6 s in total.
constexpr int kWaitPollLimit = 1 << 18;
constexpr uint32_t kWaitSuspendNs = 10000;

// ---------------------------------------------------------------- shared-memory barriers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitSuspendNs)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; gives up after kWaitPollLimit polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kWaitPollLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Bulk asynchronous copy global -> this CTA's shared memory, completion counted in bytes on
// `bar`.  Both addresses 16-byte aligned, bytes a multiple of 16.  No multicast: the
// destination is always the issuing CTA (a cluster of one).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may have its CTAs placed on
// the SMs while the kernel before it in the stream is still draining; it must not touch global memory
// before pdl_wait(), which returns once that kernel has completed and its writes are visible (at once
// when the launch carried no such attribute).  pdl_trigger() tells the scheduler that the kernel
// AFTER this one may be placed as soon as room frees up.  Both are no-ops for plain launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- strict fp32 arithmetic
// The reference materialises an fp32 tensor after every elementwise call, so products must not
// be contracted into FMAs.  The _rn intrinsics are never fused by the compiler.
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }

// Correctly rounded a / d for a fixed divisor d with dinv = RN(1/d): quotient estimate, exact
// residual by FMA, one correction (Markstein).  Equals IEEE division for finite, normal
// results; three instructions instead of the ~10 of a general division.
struct DivConst {
    float d, dinv;
    __device__ __forceinline__ float operator()(float a) const {
        float q0 = __fmul_rn(a, dinv);
        float r = __fmaf_rn(-q0, d, a);
        return __fmaf_rn(r, dinv, q0);
    }
};

// ---------------------------------------------------------------- 16-byte vectors
template <typename T>
struct Vec;  // EPV elements of T in one uint4
template <>
struct Vec<float> {
    static constexpr int EPV = 4;
    __device__ __forceinline__ static void unpack(const uint4& u, float (&f)[4]) {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    __device__ __forceinline__ static float load1(const float* p) { return *p; }
    __device__ __forceinline__ static void store1(float* p, float v) { *p = v; }
};
template <>
struct Vec<__nv_bfloat16> {
    static constexpr int EPV = 8;
    __device__ __forceinline__ static void unpack(const uint4& u, float (&f)[8]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);  // .x = low half
            w[i] = *reinterpret_cast<uint32_t*>(&b);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ __forceinline__ static void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Streaming 16-byte store: outputs are written once and not re-read by this kernel.
__device__ __forceinline__ void store_vec_streaming(void* gptr, const uint4& v) {
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(gptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// ---------------------------------------------------------------- fp64 reductions
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// rstd exactly as the reference composes it (normalization.cpp:25-26):
//   variance = reduce_mean(x*x)  -> fp32;  v = variance + eps;  s = sqrt(v);  rstd = 1.0f / s
__device__ __forceinline__ float rstd_from_sumsq(double sumsq, int hidden, float eps) {
    float var = static_cast<float>(sumsq / static_cast<double>(hidden));
    float v = __fadd_rn(var, eps);
    float s = __fsqrt_rn(v);
    return __fdiv_rn(1.0f, s);
}

}  // namespace agb
