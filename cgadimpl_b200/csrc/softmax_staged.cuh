// softmax_staged.cuh -- row softmax / logsumexp over the last axis and their rules, on the same
// skeleton as the RMSNorm kernels: persistent CTAs, rows brought into a shared-memory ring by the bulk
// asynchronous copy engine (no multicast), bounded mbarrier waits, fp64 reductions rounded once, 16-byte
// streaming stores.
//
// Rounding follows the reference's composition op by op (cgadimpl/src/ops/reduction.cpp:42-66):
//   m = max(z) ; zs = z - m (fp32) ; e = exp(zs) (fp32) ; s = (float)sum_fp64(e) ; y = e / s (IEEE fp32)
//   logsumexp = log(s) + m
// exp is evaluated to ~2^-33 relative before its one rounding to fp32 (double-word fp32 arithmetic: a
// 256-entry table of 2^(j/256) as hi + lo, an exact Cody-Waite reduction, a cubic in r), log in fp64:
// the results are the correctly rounded ones except in ~0.1 % of the cases -- the same order as a C
// library expf, whose < 1 ulp error shows up equally rarely.
#pragma once
#include <math.h>

#include "rmsnorm_fast.cuh"

namespace agb {

// ---------------------------------------------------------------- exp / log, fp64 inside
// exp(x) for x <= 0 as a float: x = (k/32) ln2 + r, |r| <= ln2/64; exp(r) by a degree-5 Taylor
// polynomial (truncation 2e-15 relative), 2^(j/32) from a 32-entry table, 2^(k>>5) by an exponent add.
constexpr int kExpTableSize = 32;
__device__ __forceinline__ void init_exp_table(double* tab) {
    if (threadIdx.x < kExpTableSize) tab[threadIdx.x] = exp2(static_cast<double>(threadIdx.x) / kExpTableSize);
}
__device__ __forceinline__ float exp_nonpositive(float x, const double* tab) {
    // below -104 the result is under half the smallest subnormal float: exactly 0 after rounding
    const double xd = static_cast<double>(fmaxf(x, -104.0f));
    const double kMagic = 6755399441055744.0;  // 1.5 * 2^52: adding it rounds to an integer in the low word
    const double t = fma(xd, 0x1.71547652b82fep+5 /* 32/ln2 */, kMagic);
    const int ki = __double2loint(t);
    const double kd = t - kMagic;
    double r = fma(kd, -0x1.62e42fe000000p-6 /* ln2/32, high 28 bits: kd * this is exact */, xd);
    r = fma(kd, -0x1.f473de6af278fp-35 /* ln2/32, rest */, r);
    double p = fma(r, 1.0 / 120.0, 1.0 / 24.0);
    p = fma(p, r, 1.0 / 6.0);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    const double s = p * tab[ki & (kExpTableSize - 1)];
    // times 2^(ki >> 5): the double stays normal (exponent >= -151), the float conversion does the rest
    const double scaled = __hiloint2double(__double2hiint(s) + (ki >> 5) * (1 << 20), __double2loint(s));
    return static_cast<float>(scaled);
}
// The fast form for -86 <= x <= 0, all in fp32 (about 16 instructions against 27 for the fp64 route, and no
// use of the fp64 / conversion pipes):
//   k = rint(x * 256/ln2);  r = (x - k*C1) - k*C2  (C1 + C2 = ln2/256; the first step is EXACT: both terms
//   are multiples of 2^-32 and their difference is below 2^-9)
//   exp(r) - 1 = w = r + r^2 (1/2 + r/6)          (|r| <= 1.36e-3; the r^4 term is 2^-43)
//   2^(j/256) = Th + Tl, j = k mod 256;  result = (Th + (Tl + Th*w)) * 2^(k div 256)
// Every rounding before the last addition is 2^-25 of a term of size 1.4e-3, i.e. ~2^-34 of the result.
constexpr int kExp32Size = 256;
__device__ __forceinline__ void init_exp32_table(float2* tab) {
    for (int j = threadIdx.x; j < kExp32Size; j += blockDim.x) {
        const double t = exp2(static_cast<double>(j) / kExp32Size);
        const float hi = static_cast<float>(t);
        tab[j] = make_float2(hi, static_cast<float>(t - static_cast<double>(hi)));
    }
}
__device__ __forceinline__ float exp_fast_range(float x, const float2* tab32) {   // -86 <= x <= 0
    const float kMagic = 12582912.0f;                    // 1.5 * 2^23, bit pattern 0x4B400000
    const float t = __fmaf_rn(x, 0x1.715476p+8f /* 256/ln2 */, kMagic);
    const int k = __float_as_int(t) - 0x4B400000;
    const float kf = __fsub_rn(t, kMagic);
    float r = __fmaf_rn(kf, -0x1.62e430p-9f /* C1 */, x);
    r = __fmaf_rn(kf, 0x1.05c610p-37f /* -C2 */, r);
    const float p = __fmaf_rn(r, 0x1.555556p-3f /* 1/6 */, 0.5f);
    const float w = __fmaf_rn(__fmul_rn(r, r), p, r);
    const float2 T = tab32[k & (kExp32Size - 1)];
    const float y = __fadd_rn(T.x, __fmaf_rn(T.x, w, T.y));
    return __int_as_float(__float_as_int(y) + (k >> 8) * (1 << 23));
}
__device__ __forceinline__ float exp_nonpositive32(float x, const float2* tab32, const double* tab64) {
    if (x < -86.0f) return exp_nonpositive(x, tab64);   // results next to or below the normal range
    return exp_fast_range(x, tab32);
}
// N values at once: one test (on their minimum) decides between the fast form for all and the fp64 route
// for all, so the common case carries one branch per vector instead of one per element.
template <int N>
__device__ __forceinline__ void exp_nonpositive32_vec(float (&f)[N], float vmin, const float2* tab32, const double* tab64) {
    if (vmin < -86.0f) {
#pragma unroll
        for (int e = 0; e < N; ++e) f[e] = exp_nonpositive(f[e], tab64);
    } else {
#pragma unroll
        for (int e = 0; e < N; ++e) f[e] = exp_fast_range(f[e], tab32);
    }
}

// The approximate form (softmax "fast" arithmetic): Cody-Waite split x = n ln2 + r, |r| <= ln2/2, then the
// hardware 2^u approximation on u = r log2(e) in [-1/2, 1/2] (2 ulp) and an exponent add; about 2e-7
// relative for -86 <= x <= 0, 0 below (results within a factor 4 of the smallest normal float, or under it, are flushed).  Eight instructions.
__device__ __forceinline__ float exp_approx_nonpositive(float x) {
    const float kMagic = 12582912.0f;                     // 1.5 * 2^23: the low mantissa bits of t hold n
    const float xc = fmaxf(x, -86.0f);
    const float t = __fmaf_rn(xc, 0x1.715476p+0f /* log2(e) */, kMagic);
    const float n = __fsub_rn(t, kMagic);
    float r = __fmaf_rn(n, -0x1.62e400p-1f /* ln2, high 15 bits: n * this is exact */, xc);
    r = __fmaf_rn(n, -0x1.7f7d1cp-20f /* ln2, rest */, r);
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(__fmul_rn(r, 0x1.715476p+0f)));
    const float y = __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
    return x < -86.0f ? 0.0f : y;
}

__device__ __forceinline__ float ex2_approx(float u) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(u));
    return p;
}

// e = exp(x - mx) for 16-bit I/O: one multiply-add and the hardware 2^u approximation, with nmx2 = -mx*log2(e)
// computed once per row.  The argument's rounding (2^-24 of |x - mx| <= 126) bounds the relative error by
// ~3e-6, three orders below the 16-bit output's own rounding; results under the normal range flush to zero.
__device__ __forceinline__ float exp_rel16(float x, float nmx2) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(__fmaf_rn(x, 0x1.715476p+0f, nmx2)));
    return p;
}

// exp(t), t <= 0, for a term of a SUM (logsumexp): the hardware 2^u on t*log2(e).  Relative error about
// 2.4e-7 + 1.2e-7*|t|: the terms that matter to the sum (t near 0) are as good as the careful form's, the
// others are wrong by a little more in proportion to how little they matter; under the normal range it flushes.
__device__ __forceinline__ float exp_for_sum(float t) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(__fmul_rn(t, 0x1.715476p+0f)));
    return p;
}

// max of two packed bf16 pairs, lane by lane (a NaN lane yields the other operand, like fmaxf)
__device__ __forceinline__ uint32_t packed_max(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// e = exp(z - mx) for one vector, in place, and its contribution to four fp32 sum chains
template <typename T>
__device__ __forceinline__ void exp_fast_vec(float (&f)[Vec<T>::EPV], float mx, float nmx2, float& a0, float& a1, float& a2,
                                             float& a3) {
    constexpr int EPV = Vec<T>::EPV;
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
        if constexpr (sizeof(T) == 2) f[e] = exp_rel16(f[e], nmx2);
        else f[e] = exp_approx_nonpositive(f[e] - mx);
    }
#pragma unroll
    for (int e = 0; e < EPV; e += 4) {
        a0 += f[e]; a1 += f[e + 1]; a2 += f[e + 2]; a3 += f[e + 3];
    }
}

__device__ __forceinline__ float log_rounded(float s) { return static_cast<float>(log(static_cast<double>(s))); }

// a / d for one divisor per row (1 <= d <= 2^24, 0 <= a <= 1).  `fast` is the three-instruction exact
// division of DivConst; it needs the residual a - q0*d to be free of underflow, which holds for
// a == 0 and for a >= exp(-40) (q0 >= 2^-82: the residual's granule 2^-128 is representable).  Rows
// that contain smaller non-zero numerators (masked logits) go through `guarded`, element by element.
constexpr float kRowDivSafeShift = -40.0f;  // z - max below this makes the row take the guarded path
struct RowDiv {
    float d, dinv;
    __device__ __forceinline__ float fast(float a) const {
        const float q0 = __fmul_rn(a, dinv);
        const float r = __fmaf_rn(-q0, d, a);
        return __fmaf_rn(r, dinv, q0);
    }
    __device__ __forceinline__ float guarded(float a) const {
        const float q0 = __fmul_rn(a, dinv);
        if (!(q0 > 1e-30f && q0 < 1e30f)) return __fdiv_rn(a, d);
        const float r = __fmaf_rn(-q0, d, a);
        return __fmaf_rn(r, dinv, q0);
    }
};

struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };
__device__ __forceinline__ RowDiv make_row_div(float divisor) { return RowDiv{divisor, __frcp_rn(divisor)}; }

__device__ __forceinline__ void fence_generic_to_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float group_max(const float* s_red, int wpr, int lane) {
    return warp_max(lane < wpr ? s_red[lane] : -INFINITY);
}

// ------------------------------------------------------------------------------------------
// Forward family.  MODE 0: out = softmax(z).  1: out_row = logsumexp(z).  2: out = rowscale * softmax(z)
// [+ add]  (the logsumexp VJP).  3: out_row = sum(softmax(z) * t)  (the logsumexp JVP; t is staged next
// to z).  e is parked in shared memory between the passes: in place over z for fp32, in a scratch
// region of the stage (two row-widths) for bf16.
// ------------------------------------------------------------------------------------------
struct SoftmaxArgs {
    PipeGeom g;
    const void* z;
    const void* t;         // MODE 3
    const void* rowscale;  // MODE 2: [rows] of T
    const void* add;       // MODE 2, nullable: [rows, hidden] added to the result (gradient accumulation)
    void* out;             // [rows, hidden]
    void* out_row;         // [rows] of T
    int scratch_offset;    // bytes from the start of a stage to the fp32 scratch (0: in place over z)
};

// FAST: exp by exp_approx_nonpositive, sums in fp32, y = e * (1/s) -- about 2e-7 relative per element, far
// inside the path's rel 1e-5, at under half the instructions of the strictly rounded form (which reproduces
// the reference composition's bits and stays available through the "softmax_strict" option).
// KV > 0 (FAST only): every thread owns at most KV vectors of its row and keeps their e in registers between
// the passes instead of parking them in shared memory (no scratch region, one shared-memory round trip less).
template <typename T, int MODE, bool FAST, int KV = 0>
__global__ void __launch_bounds__(1024, 1) softmax_fwd_staged(const __grid_constant__ SoftmaxArgs a) {
    static_assert(KV == 0 || FAST, "registers keep e only in the approximate form");
    constexpr int EPV = Vec<T>::EPV;
    constexpr int NARR = MODE == 3 ? 2 : 1;
    constexpr bool kThreePasses = MODE != 1;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ double s_exp[kExpTableSize];
    __shared__ float2 s_exp32[kExp32Size];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    init_exp_table(s_exp);
    init_exp32_table(s_exp32);
    __syncthreads();

    const unsigned char* const src2[2] = {reinterpret_cast<const unsigned char*>(a.z),
                                          reinterpret_cast<const unsigned char*>(a.t)};
    auto issue = [&](long long tile, int slot) {
        if (NARR == 2) issue_tile<2>(g, ring, s_full, src2, tile, slot);
        else issue_tile<1>(g, ring, s_full, reinterpret_cast<const unsigned char* const(&)[1]>(src2), tile, slot);
    };
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued) issue(first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;

        unsigned char* stage = ring + static_cast<size_t>(slot) * g.stage_stride;
        const uint4* sz = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(grp) * g.row_bytes);
        const uint4* st = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sz) + g.tile_stride);
        // fp32 e of this row: EPV floats (EPV/4 vectors) per input vector
        float4* se = a.scratch_offset
                         ? reinterpret_cast<float4*>(stage + a.scratch_offset + static_cast<size_t>(grp) * g.hidden * 4)
                         : reinterpret_cast<float4*>(stage + static_cast<size_t>(grp) * g.row_bytes);
        double* red = s_red + (k & 1) * 4 * nwarps;
        float* redf = reinterpret_cast<float*>(red);

        // pass 1: row maximum
        float m = -INFINITY;
        if (valid)
            for (int v = tig; v < g.nvec; v += G) {
                float f[EPV];
                Vec<T>::unpack(sz[v], f);
#pragma unroll
                for (int e = 0; e < EPV; ++e) m = fmaxf(m, f[e]);
            }
        m = warp_max(m);
        if (lane == 0) redf[warp] = m;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // every thread is past the last pass of the previous tile: its slot can be refilled
        if (kThreePasses && tid == 0 && k >= 1 && issued < my_tiles) {
            issue(first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float mx = group_max(redf + grp * wpr, wpr, lane);

        // pass 2: e = exp(z - max), its sum in fp64; `tiny`: some z - max is so low that the fast
        // division of pass 3 would not be exact
        double d0 = 0.0, d1 = 0.0;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;   // FAST: four fp32 chains
        float keep[KV > 0 ? KV * EPV : 1];
        const float nmx2 = -mx * 0x1.715476p+0f;
        bool tiny = false;
        if constexpr (KV > 0) {
            if (valid) {
#pragma unroll
                for (int i = 0; i < KV; ++i) {
                    const int v = tig + i * G;
                    if (v < g.nvec) {
                        float f[EPV];
                        Vec<T>::unpack(sz[v], f);
                        exp_fast_vec<T>(f, mx, nmx2, a0, a1, a2, a3);
#pragma unroll
                        for (int e = 0; e < EPV; ++e) keep[i * EPV + e] = f[e];
                    }
                }
            }
        } else if (valid)
            for (int v = tig; v < g.nvec; v += G) {
                float f[EPV];
                Vec<T>::unpack(sz[v], f);
                if constexpr (FAST) {
                    exp_fast_vec<T>(f, mx, nmx2, a0, a1, a2, a3);
                } else {
                float vmin = 0.0f;
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    f[e] = sub_rn(f[e], mx);
                    vmin = fminf(vmin, f[e]);
                }
                tiny |= vmin < kRowDivSafeShift;
                exp_nonpositive32_vec<EPV>(f, vmin, s_exp32, s_exp);
#pragma unroll
                for (int e = 0; e < EPV; e += 2) {
                    d0 += static_cast<double>(f[e]);
                    d1 += static_cast<double>(f[e + 1]);
                }
                }
                if (kThreePasses) {
#pragma unroll
                    for (int q = 0; q < EPV / 4; ++q)
                        se[v * (EPV / 4) + q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
                }
            }
        (void)keep;
        const double dsum = FAST ? static_cast<double>(warp_sum_f32((a0 + a1) + (a2 + a3))) : warp_sum(d0 + d1);
        const bool warp_tiny = __any_sync(0xffffffffu, tiny);
        if (lane == 0) {
            red[nwarps + warp] = dsum;
            redf[nwarps + warp] = warp_tiny ? 1.0f : 0.0f;  // second half of the max region
        }
        if (kThreePasses && KV == 0) fence_generic_to_async_smem();  // the slot this thread wrote is refilled by the copy engine later
        __syncthreads();
        if (!kThreePasses && tid == 0 && issued < my_tiles) {  // nobody reads the slot again
            issue(first + issued * stride, slot);
            ++issued;
        }
        float s = static_cast<float>(group_total(red + nwarps + grp * wpr, wpr, lane));
        // an infinite row maximum makes z - max NaN in the composition; the clamped approximate exp would hide it
        if (FAST && fabsf(mx) == INFINITY) s = __int_as_float(0x7fc00000);
        const bool row_tiny = __any_sync(0xffffffffu, lane < wpr && redf[nwarps + grp * wpr + lane] != 0.0f);

        if (MODE == 1) {
            if (valid && tig == 0) Vec<T>::store1(static_cast<T*>(a.out_row) + row, add_rn(log_rounded(s), mx));
            continue;
        }

        // pass 3: y = e / s and what the mode makes of it
        const RowDiv div_s = make_row_div(s);
        const float scale = (MODE == 2 && valid) ? Vec<T>::load1(static_cast<const T*>(a.rowscale) + row) : 0.0f;
        const float fast_mul = FAST ? (MODE == 2 ? scale * div_s.dinv : div_s.dinv) : 0.0f;   // y (or scale*y) = e * this
        double j0 = 0.0, j1 = 0.0;
        float jf0 = 0.0f, jf1 = 0.0f;
        if (valid) {
            uint4* gout = MODE == 3 ? nullptr : reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.out) + row * g.row_bytes);
            const uint4* gadd = (MODE == 2 && a.add)
                                    ? reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.add) + row * g.row_bytes)
                                    : nullptr;
            // what becomes of one vector of e (in f): y = e / s and the mode's use of it
            auto finish_vec = [&](int v, float (&f)[EPV], bool guarded) {
                {
                    if constexpr (FAST) {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) f[e] = f[e] * fast_mul;
                    } else {
                    if (guarded) {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) f[e] = div_s.guarded(f[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) f[e] = div_s.fast(f[e]);
                    }
                    }
                    if (MODE == 2) {
                        if constexpr (!FAST) {
#pragma unroll
                        for (int e = 0; e < EPV; ++e) f[e] = mul_rn(scale, f[e]);
                        }
                        if (gadd) {
                            float ad[EPV];
                            Vec<T>::unpack(gadd[v], ad);
#pragma unroll
                            for (int e = 0; e < EPV; ++e) f[e] = add_rn(ad[e], f[e]);
                        }
                    }
                    if (MODE == 3) {
                        float tv[EPV];
                        Vec<T>::unpack(st[v], tv);
                        if constexpr (FAST) {
#pragma unroll
                            for (int e = 0; e < EPV; e += 2) {
                                jf0 = fmaf(f[e], tv[e], jf0);
                                jf1 = fmaf(f[e + 1], tv[e + 1], jf1);
                            }
                        } else {
#pragma unroll
                        for (int e = 0; e < EPV; e += 2) {
                            j0 += static_cast<double>(mul_rn(f[e], tv[e]));
                            j1 += static_cast<double>(mul_rn(f[e + 1], tv[e + 1]));
                        }
                        }
                    } else {
                        store_vec_streaming(gout + v, Vec<T>::pack(f));
                    }
                }
            };
            auto pass3 = [&](bool guarded) {
                for (int v = tig; v < g.nvec; v += G) {
                    float f[EPV];
#pragma unroll
                    for (int q = 0; q < EPV / 4; ++q) {
                        const float4 e4 = se[v * (EPV / 4) + q];
                        f[4 * q] = e4.x; f[4 * q + 1] = e4.y; f[4 * q + 2] = e4.z; f[4 * q + 3] = e4.w;
                    }
                    finish_vec(v, f, guarded);
                }
            };
            if constexpr (KV > 0) {
#pragma unroll
                for (int i = 0; i < KV; ++i) {
                    const int v = tig + i * G;
                    if (v < g.nvec) {
                        float f[EPV];
#pragma unroll
                        for (int e = 0; e < EPV; ++e) f[e] = keep[i * EPV + e];
                        finish_vec(v, f, false);
                    }
                }
            } else pass3(row_tiny);
        }
        if (MODE == 3) {
            const double jsum = FAST ? static_cast<double>(warp_sum_f32(jf0 + jf1)) : warp_sum(j0 + j1);
            if (lane == 0) red[2 * nwarps + warp] = jsum;
            __syncthreads();
            const float tot = static_cast<float>(group_total(red + 2 * nwarps + grp * wpr, wpr, lane));
            if (valid && tig == 0) Vec<T>::store1(static_cast<T*>(a.out_row) + row, tot);
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

// ------------------------------------------------------------------------------------------
// Forward in ONE pass over the staged row (approximate arithmetic only; MODE 0 softmax, 1 logsumexp).
// Every thread owns at most KV vectors of its row.  It reads them once, takes ITS OWN maximum m_t, forms
// e = exp(z - m_t) and their sum s_t in registers, and only then meets the rest of the row: the pairs (m, s)
// are merged by  M = max m,  S = sum s * exp(m - M)  inside the warp and, through shared memory, across the
// row's warps.  The result is y = e * (exp(m_t - M) / S), or log(S) + M.  One shared-memory pass and one
// block-wide barrier per tile instead of two each, and the slot is free for its refill at that barrier.
// A thread whose values are all -inf contributes nothing; a row whose maximum is infinite yields NaN, as the
// composition does (z - max is NaN there).
// ------------------------------------------------------------------------------------------
template <typename T, int MODE, int KV>
__global__ void __launch_bounds__(1024, 1) softmax_fwd_online(const __grid_constant__ SoftmaxArgs a) {
    static_assert(MODE == 0 || MODE == 1, "softmax or logsumexp");
    constexpr int EPV = Vec<T>::EPV;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    float2* s_red = reinterpret_cast<float2*>(smem + g.off_red);   // [2 tiles in turn][nwarps] of (max, sum)
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;
    constexpr float kLog2e = 0x1.715476p+0f;
    // the factor exp(m - M) of a merge: it scales a SUM in the logsumexp, an output element in the softmax
    auto merge_exp = [](float t) { return MODE == 1 ? exp_for_sum(t) : exp_approx_nonpositive(t); };

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const unsigned char* const src1[1] = {reinterpret_cast<const unsigned char*>(a.z)};
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued) issue_tile<1>(g, ring, s_full, src1, first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const uint4* sz = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes);

        float f[KV * EPV];
        float m = -INFINITY;
        uint32_t mp = 0xFF80FF80u;   // 16-bit I/O: the maximum is taken on the packed pairs, two values per instruction
#pragma unroll
        for (int i = 0; i < KV; ++i) {
            const int v = tig + i * G;
            if (valid && v < g.nvec) {
                const uint4 raw = sz[v];
                float t[EPV];
                Vec<T>::unpack(raw, t);
                if constexpr (sizeof(T) == 2) {
                    mp = packed_max(packed_max(mp, raw.x), packed_max(raw.y, packed_max(raw.z, raw.w)));
                } else {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) m = fmaxf(m, t[e]);
                }
#pragma unroll
                for (int e = 0; e < EPV; ++e) f[i * EPV + e] = t[e];
            } else {
#pragma unroll
                for (int e = 0; e < EPV; ++e) f[i * EPV + e] = -INFINITY;
            }
        }
        if constexpr (sizeof(T) == 2) m = fmaxf(__uint_as_float(mp << 16), __uint_as_float(mp & 0xffff0000u));
        const float ms = m == -INFINITY ? 0.0f : m;    // the shift this thread uses (a thread of -inf shifts by 0: e = 0)
        const float nms2 = -ms * kLog2e;
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        if constexpr (sizeof(T) == 2) {
            // 16-bit I/O: the exponent's multiply-add and the sums as packed two-lane instructions (the two values
            // of a 32-bit input word sit in neighbouring registers anyway); only the 2^u itself is per element
            const float2 l2 = make_float2(kLog2e, kLog2e), n2 = make_float2(nms2, nms2);
            float2 p0 = make_float2(0.f, 0.f), p1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < KV * EPV; i += 4) {
                const float2 u0 = __ffma2_rn(make_float2(f[i], f[i + 1]), l2, n2);
                const float2 u1 = __ffma2_rn(make_float2(f[i + 2], f[i + 3]), l2, n2);
                f[i] = ex2_approx(u0.x); f[i + 1] = ex2_approx(u0.y);
                f[i + 2] = ex2_approx(u1.x); f[i + 3] = ex2_approx(u1.y);
                p0 = __fadd2_rn(p0, make_float2(f[i], f[i + 1]));
                p1 = __fadd2_rn(p1, make_float2(f[i + 2], f[i + 3]));
            }
            a0 = p0.x; a1 = p0.y; a2 = p1.x; a3 = p1.y;
        } else {
#pragma unroll
            for (int i = 0; i < KV * EPV; i += 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if constexpr (MODE == 1) f[i + e] = exp_for_sum(f[i + e] - ms);
                    else f[i + e] = exp_approx_nonpositive(f[i + e] - ms);
                }
                a0 += f[i]; a1 += f[i + 1]; a2 += f[i + 2]; a3 += f[i + 3];
            }
        }
        const float st = (a0 + a1) + (a2 + a3);
        // merge inside the warp
        const float mw = warp_max(m);
        const float mws = mw == -INFINITY ? 0.0f : mw;
        const float sw = warp_sum_f32(m == -INFINITY ? 0.0f : st * merge_exp(ms - mws));
        float2* red = s_red + (k & 1) * nwarps;
        if (lane == 0) red[warp] = make_float2(mw, sw);
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        // every thread holds its part of the tile in registers: the slot can be refilled now
        if (tid == 0 && issued < my_tiles) {
            issue_tile<1>(g, ring, s_full, src1, first + issued * stride, slot);
            ++issued;
        }
        // merge the row's warps (every thread of the row computes the same M and S)
        float M = mw, Ssum = sw;
        if (wpr > 1) {
            const float2 p = lane < wpr ? red[grp * wpr + lane] : make_float2(-INFINITY, 0.0f);
            M = warp_max(p.x);
            const float Msafe = M == -INFINITY ? 0.0f : M;
            Ssum = warp_sum_f32(p.x == -INFINITY ? 0.0f : p.y * merge_exp(p.x - Msafe));
        }
        const float Ms = M == -INFINITY ? 0.0f : M;
        const float nan = __int_as_float(0x7fc00000);
        if (MODE == 1) {
            if (valid && tig == 0)
                Vec<T>::store1(static_cast<T*>(a.out_row) + row, fabsf(M) == INFINITY ? nan : logf(Ssum) + M);
            continue;
        }
        const float c = fabsf(M) == INFINITY ? nan : (m == -INFINITY ? 0.0f : exp_approx_nonpositive(ms - Ms) * __frcp_rn(Ssum));
        if (valid) {
            uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.out) + row * g.row_bytes);
#pragma unroll
            for (int i = 0; i < KV; ++i) {
                const int v = tig + i * G;
                if (v < g.nvec) {
                    float t[EPV];
#pragma unroll
                    for (int e = 0; e < EPV; ++e) t[e] = f[i * EPV + e] * c;
                    store_vec_streaming(gout + v, Vec<T>::pack(t));
                }
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

// ------------------------------------------------------------------------------------------
// out = y * (g - sum(y * g)) [+ add]: the softmax VJP (g = gy) and JVP (g = tangent),
// cgadimpl/src/autodiff/autodiff_vjp_ops.cpp:421-428 and autodiff_jvp_ops.cpp:411-420.
// ------------------------------------------------------------------------------------------
struct SoftmaxBwdArgs {
    PipeGeom g;
    const void* y;
    const void* gr;
    const void* add;  // nullable
    void* out;
};

template <typename T>
__global__ void __launch_bounds__(1024, 1) softmax_bwd_staged(const __grid_constant__ SoftmaxBwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    extern __shared__ __align__(128) unsigned char smem[];
    const PipeGeom& g = a.g;
    unsigned char* ring = smem;
    double* s_red = reinterpret_cast<double*>(smem + g.off_red);
    uint64_t* s_full = reinterpret_cast<uint64_t*>(smem + g.off_bar);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + g.off_flag);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int G = g.group_threads, wpr = G >> 5;
    const int grp = tid / G, tig = tid - grp * G;
    const int S = g.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(&s_full[s], 1);
        *s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const unsigned char* const src2[2] = {reinterpret_cast<const unsigned char*>(a.y),
                                          reinterpret_cast<const unsigned char*>(a.gr)};
    const long long first = blockIdx.x, stride = gridDim.x;
    const long long my_tiles = g.ntiles > first ? (g.ntiles - first + stride - 1) / stride : 0;
    long long issued = 0;
    if (tid == 0)
        for (; issued < my_tiles && issued < S; ++issued)
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>(issued));

    long long k = 0;
    bool aborted = false;
    for (; k < my_tiles; ++k) {
        const int slot = static_cast<int>(k % S);
        const uint32_t parity = static_cast<uint32_t>((k / S) & 1);
        const long long row = (first + k * stride) * g.rows_per_tile + grp;
        const bool valid = row < g.rows;
        if (!mbar_wait_bounded(&s_full[slot], parity)) *s_abort = 1;
        const unsigned char* base = ring + static_cast<size_t>(slot) * g.stage_stride + static_cast<size_t>(grp) * g.row_bytes;
        const uint4* sy = reinterpret_cast<const uint4*>(base);
        const uint4* sg = reinterpret_cast<const uint4*>(base + g.tile_stride);

        double d[4] = {0.0, 0.0, 0.0, 0.0};
        if (valid) {
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 yv[NP], gv[NP];
                Pairs<T>::unpack(sy[v], yv);
                Pairs<T>::unpack(sg[v], gv);
#pragma unroll
                for (int e = 0; e < NP; ++e) {
                    const float2 p = mul2(yv[e], gv[e]);
                    d[(2 * e) & 3] += static_cast<double>(p.x);
                    d[(2 * e + 1) & 3] += static_cast<double>(p.y);
                }
            }
        }
        const double dsum = warp_sum((d[0] + d[1]) + (d[2] + d[3]));
        if (lane == 0) s_red[(k & 1) * nwarps + warp] = dsum;
        __syncthreads();
        if (*s_abort) { aborted = true; break; }
        if (tid == 0 && k >= 1 && issued < my_tiles) {
            issue_tile<2>(g, ring, s_full, src2, first + issued * stride, static_cast<int>((k - 1) % S));
            ++issued;
        }
        const float dot = static_cast<float>(group_total(s_red + (k & 1) * nwarps + grp * wpr, wpr, lane));
        const float2 dot2 = splat(dot);

        if (valid) {
            uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.out) + row * g.row_bytes);
            const uint4* gadd =
                a.add ? reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.add) + row * g.row_bytes) : nullptr;
#pragma unroll 2
            for (int v = tig; v < g.nvec; v += G) {
                float2 yv[NP], gv[NP];
                Pairs<T>::unpack(sy[v], yv);
                Pairs<T>::unpack(sg[v], gv);
#pragma unroll
                for (int e = 0; e < NP; ++e) yv[e] = mul2(yv[e], sub2(gv[e], dot2));  // g - dot: neither is a product
                if (gadd) {
                    float2 av[NP];
                    Pairs<T>::unpack(gadd[v], av);
#pragma unroll
                    for (int e = 0; e < NP; ++e) yv[e] = add2_after_mul(av[e], yv[e]);
                }
                store_vec_streaming(gout + v, Pairs<T>::pack(yv));
            }
        }
    }
    if (aborted && tid == 0) drain_after_abort(g, s_full, k, issued);
}

// ------------------------------------------------------------------------------------------
// Rows too wide for the shared-memory ring (vocabulary-sized logits) but 16-byte aligned: one CTA of
// 1024 threads per row, 16-byte loads, three passes over the row of which only the first comes from DRAM
// (a row is at most 1 MB and stays in L2); e is recomputed in the last pass instead of being parked.
// Same modes and the same bits as softmax_fwd_staged.
// ------------------------------------------------------------------------------------------
constexpr int kWideThreads = 1024;
__device__ __forceinline__ uint4 ldg128(const uint4* p) { return __ldg(p); }

template <typename T, int MODE>
__global__ void __launch_bounds__(kWideThreads, 1) softmax_fwd_wide(const __grid_constant__ SoftmaxArgs a) {
    constexpr int EPV = Vec<T>::EPV;
    __shared__ double s_exp[kExpTableSize];
    __shared__ float2 s_exp32[kExp32Size];
    __shared__ double s_redd[2][32];
    __shared__ float s_redf[2][64];
    const PipeGeom& g = a.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int nwarps = kWideThreads / 32;
    init_exp_table(s_exp);
    init_exp32_table(s_exp32);
    __syncthreads();
    int phase = 0;
    for (long long row = blockIdx.x; row < g.rows; row += gridDim.x, phase ^= 1) {
        const uint4* zr = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.z) + row * g.row_bytes);
        // pass 1: maximum
        float m = -INFINITY;
#pragma unroll 4
        for (int v = tid; v < g.nvec; v += kWideThreads) {   // unrolled: several 16-byte loads in flight per thread
            float f[EPV];
            Vec<T>::unpack(ldg128(zr + v), f);
#pragma unroll
            for (int e = 0; e < EPV; ++e) m = fmaxf(m, f[e]);
        }
        m = warp_max(m);
        if (lane == 0) s_redf[phase][warp] = m;
        __syncthreads();
        const float mx = warp_max(s_redf[phase][lane]);   // nwarps == 32
        // pass 2: sum of exp, and whether the fast division is exact for this row
        double d0 = 0.0, d1 = 0.0;
        bool tiny = false;
#pragma unroll 2
        for (int v = tid; v < g.nvec; v += kWideThreads) {
            float f[EPV];
            Vec<T>::unpack(ldg128(zr + v), f);
            float vmin = 0.0f;
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                f[e] = sub_rn(f[e], mx);
                vmin = fminf(vmin, f[e]);
            }
            tiny |= vmin < kRowDivSafeShift;
            exp_nonpositive32_vec<EPV>(f, vmin, s_exp32, s_exp);
#pragma unroll
            for (int e = 0; e < EPV; e += 2) {
                d0 += static_cast<double>(f[e]);
                d1 += static_cast<double>(f[e + 1]);
            }
        }
        const double dsum = warp_sum(d0 + d1);
        const bool warp_tiny = __any_sync(0xffffffffu, tiny);
        if (lane == 0) {
            s_redd[phase][warp] = dsum;
            s_redf[phase][32 + warp] = warp_tiny ? 1.0f : 0.0f;
        }
        __syncthreads();
        const float s = static_cast<float>(warp_sum(s_redd[phase][lane]));
        const bool row_tiny = __any_sync(0xffffffffu, s_redf[phase][32 + lane] != 0.0f);
        if (MODE == 1) {
            if (tid == 0) Vec<T>::store1(static_cast<T*>(a.out_row) + row, add_rn(log_rounded(s), mx));
            continue;
        }
        // pass 3
        const RowDiv div_s = make_row_div(s);
        const float scale = MODE == 2 ? Vec<T>::load1(static_cast<const T*>(a.rowscale) + row) : 0.0f;
        uint4* gout = MODE == 3 ? nullptr : reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.out) + row * g.row_bytes);
        const uint4* gadd = (MODE == 2 && a.add) ? reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.add) + row * g.row_bytes) : nullptr;
        const uint4* tr = MODE == 3 ? reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.t) + row * g.row_bytes) : nullptr;
        double j0 = 0.0, j1 = 0.0;
#pragma unroll 2
        for (int v = tid; v < g.nvec; v += kWideThreads) {
            float f[EPV];
            Vec<T>::unpack(ldg128(zr + v), f);
            float vmin = 0.0f;
#pragma unroll
            for (int e = 0; e < EPV; ++e) {
                f[e] = sub_rn(f[e], mx);
                vmin = fminf(vmin, f[e]);
            }
            exp_nonpositive32_vec<EPV>(f, vmin, s_exp32, s_exp);
            if (row_tiny) {
#pragma unroll
                for (int e = 0; e < EPV; ++e) f[e] = div_s.guarded(f[e]);
            } else {
#pragma unroll
                for (int e = 0; e < EPV; ++e) f[e] = div_s.fast(f[e]);
            }
            if (MODE == 2) {
#pragma unroll
                for (int e = 0; e < EPV; ++e) f[e] = mul_rn(scale, f[e]);
                if (gadd) {
                    float ad[EPV];
                    Vec<T>::unpack(gadd[v], ad);   // may alias the output: plain load
#pragma unroll
                    for (int e = 0; e < EPV; ++e) f[e] = add_rn(ad[e], f[e]);
                }
            }
            if (MODE == 3) {
                float tv[EPV];
                Vec<T>::unpack(ldg128(tr + v), tv);
#pragma unroll
                for (int e = 0; e < EPV; e += 2) {
                    j0 += static_cast<double>(mul_rn(f[e], tv[e]));
                    j1 += static_cast<double>(mul_rn(f[e + 1], tv[e + 1]));
                }
            } else {
                store_vec_streaming(gout + v, Vec<T>::pack(f));
            }
        }
        if (MODE == 3) {
            const double jsum = warp_sum(j0 + j1);
            __syncthreads();   // everyone has read s_redd[phase] of pass 2
            if (lane == 0) s_redd[phase][warp] = jsum;
            __syncthreads();
            const float tot = static_cast<float>(warp_sum(s_redd[phase][lane]));
            if (tid == 0) Vec<T>::store1(static_cast<T*>(a.out_row) + row, tot);
        }
    }
}

// The same for out = y * (g - sum(y*g)) [+ add].
template <typename T>
__global__ void __launch_bounds__(kWideThreads, 1) softmax_bwd_wide(const __grid_constant__ SoftmaxBwdArgs a) {
    constexpr int NP = Pairs<T>::NP;
    __shared__ double s_redd[2][32];
    const PipeGeom& g = a.g;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int phase = 0;
    for (long long row = blockIdx.x; row < g.rows; row += gridDim.x, phase ^= 1) {
        const uint4* yr = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.y) + row * g.row_bytes);
        const uint4* gr = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.gr) + row * g.row_bytes);
        double d[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll 2
        for (int v = tid; v < g.nvec; v += kWideThreads) {
            float2 yv[NP], gv[NP];
            Pairs<T>::unpack(ldg128(yr + v), yv);
            Pairs<T>::unpack(ldg128(gr + v), gv);
#pragma unroll
            for (int e = 0; e < NP; ++e) {
                const float2 p = mul2(yv[e], gv[e]);
                d[(2 * e) & 3] += static_cast<double>(p.x);
                d[(2 * e + 1) & 3] += static_cast<double>(p.y);
            }
        }
        const double dsum = warp_sum((d[0] + d[1]) + (d[2] + d[3]));
        if (lane == 0) s_redd[phase][warp] = dsum;
        __syncthreads();
        const float2 dot2 = splat(static_cast<float>(warp_sum(s_redd[phase][lane])));
        uint4* gout = reinterpret_cast<uint4*>(static_cast<unsigned char*>(a.out) + row * g.row_bytes);
        const uint4* gadd = a.add ? reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.add) + row * g.row_bytes) : nullptr;
#pragma unroll 2
        for (int v = tid; v < g.nvec; v += kWideThreads) {
            float2 yv[NP], gv[NP];
            Pairs<T>::unpack(ldg128(yr + v), yv);
            Pairs<T>::unpack(ldg128(gr + v), gv);
#pragma unroll
            for (int e = 0; e < NP; ++e) yv[e] = mul2(yv[e], sub2(gv[e], dot2));
            if (gadd) {
                float2 av[NP];
                Pairs<T>::unpack(gadd[v], av);   // may alias the output: plain load
#pragma unroll
                for (int e = 0; e < NP; ++e) yv[e] = add2_after_mul(av[e], yv[e]);
            }
            store_vec_streaming(gout + v, Pairs<T>::pack(yv));
        }
    }
}

// ------------------------------------------------------------------------------------------
// Unstaged versions: any hidden size, element-aligned pointers.  One CTA of 256 threads per row;
// e is recomputed in the last pass instead of being parked (same bits: exp is a pure function).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_max_256(float v, float* scratch, int phase) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    float* s = scratch + (phase & 1) * 8;
    if (lane == 0) s[warp] = v;
    __syncthreads();
    float t = s[0];
#pragma unroll
    for (int w = 1; w < kGenericThreads / 32; ++w) t = fmaxf(t, s[w]);
    return t;
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kGenericThreads) softmax_fwd_generic(const T* __restrict__ z, const T* __restrict__ t,
                                                                       const T* __restrict__ rowscale, const T* add,
                                                                       T* out, T* __restrict__ out_row, long long rows,
                                                                       int hidden) {
    __shared__ double scratch[32];
    __shared__ float scratch_f[16];
    __shared__ double s_exp[kExpTableSize];
    __shared__ float2 s_exp32[kExp32Size];
    init_exp_table(s_exp);
    init_exp32_table(s_exp32);
    __syncthreads();
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++phase) {
        const T* zr = z + row * hidden;
        float m = -INFINITY;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) m = fmaxf(m, Vec<T>::load1(zr + j));
        const float mx = block_max_256(m, scratch_f, phase);
        double d = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads)
            d += static_cast<double>(exp_nonpositive32(sub_rn(Vec<T>::load1(zr + j), mx), s_exp32, s_exp));
        const float s = static_cast<float>(block_sum_256(d, scratch, phase));
        if (MODE == 1) {
            if (threadIdx.x == 0) Vec<T>::store1(out_row + row, add_rn(log_rounded(s), mx));
            continue;
        }
        const RowDiv div_s = make_row_div(s);
        const float scale = MODE == 2 ? Vec<T>::load1(rowscale + row) : 0.0f;
        double jd = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            float y = div_s.guarded(exp_nonpositive32(sub_rn(Vec<T>::load1(zr + j), mx), s_exp32, s_exp));
            if (MODE == 2) {
                y = mul_rn(scale, y);
                if (add) y = add_rn(Vec<T>::load1(add + row * hidden + j), y);
            }
            if (MODE == 3) jd += static_cast<double>(mul_rn(y, Vec<T>::load1(t + row * hidden + j)));
            else Vec<T>::store1(out + row * hidden + j, y);
        }
        if (MODE == 3) {
            const float tot = static_cast<float>(block_sum_256(jd, scratch + 16, phase));
            if (threadIdx.x == 0) Vec<T>::store1(out_row + row, tot);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads) softmax_bwd_generic(const T* __restrict__ y, const T* __restrict__ gr,
                                                                       const T* add, T* out, long long rows, int hidden) {
    __shared__ double scratch[16];
    int phase = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++phase) {
        const T* yr = y + row * hidden;
        const T* gg = gr + row * hidden;
        double d = 0.0;
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads)
            d += static_cast<double>(mul_rn(Vec<T>::load1(yr + j), Vec<T>::load1(gg + j)));
        const float dot = static_cast<float>(block_sum_256(d, scratch, phase));
        for (int j = threadIdx.x; j < hidden; j += kGenericThreads) {
            float o = mul_rn(Vec<T>::load1(yr + j), sub_rn(Vec<T>::load1(gg + j), dot));
            if (add) o = add_rn(Vec<T>::load1(add + row * hidden + j), o);
            Vec<T>::store1(out + row * hidden + j, o);
        }
    }
}

}  // namespace agb
