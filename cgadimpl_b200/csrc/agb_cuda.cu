// agb_cuda.cu -- the C ABI of libagb_cuda.so (declared in include/agb/agb.h) and the launch
// heuristics behind it.  Single translation unit: all kernels are included here.
#include "agb/agb.h"

#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "agb_device.cuh"
#include "elementwise.cuh"
#include "rmsnorm_generic.cuh"
#include "rmsnorm_staged.cuh"
#include "rmsnorm_fast.cuh"
#include "layernorm_staged.cuh"
#include "softmax_staged.cuh"
#include "agb_peer_device.cuh"

namespace {

using agb::PipeGeom;
typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------ errors
thread_local char t_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    return fail(AGB_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}
#define AGB_CUDA(call)                                     \
    do {                                                   \
        cudaError_t e__ = (call);                          \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
    } while (0)

std::atomic<uint64_t> g_launches{0};

// An NVTX range around every compute entry point, so that a timeline tool shows which C-ABI call enqueued
// which kernels (header-only NVTX 3: a no-op costing a few nanoseconds when no tool is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};
#define AGB_RANGE() NvtxRange nvtx_range__(__func__)

int after_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return AGB_OK;
}

// ------------------------------------------------------------------ device properties
struct DevInfo {
    int sms = 0;
    int smem_optin = 0;   // max dynamic shared memory per block
    int smem_per_sm = 0;
    bool ok = false;
};
constexpr int kMaxDevices = 64;
DevInfo g_dev[kMaxDevices];
std::mutex g_dev_mu;

int device_info(const DevInfo** out) {
    int dev = 0;
    AGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(AGB_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    DevInfo& d = g_dev[dev];
    if (!d.ok) {
        AGB_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
        AGB_CUDA(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        AGB_CUDA(cudaDeviceGetAttribute(&d.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
        d.ok = true;
    }
    *out = &d;
    return AGB_OK;
}

// ------------------------------------------------------------------ options
std::atomic<int64_t> opt_stages{0}, opt_ctas_per_sm{0}, opt_threads{0}, opt_force_generic{0}, opt_ept{0}, opt_rpw{0};
// bf16_strict: 16-bit I/O through the strictly rounded fp64-reducing kernels instead of the fp32-accumulating ones.
// bwd_keep: fast backward variant (0 auto, 1 registers keep x and gy between the passes, 2 re-read the tile).
// reserve_sms: SMs the persistent grids leave free (for a collective's kernel running beside them).
// pdl: programmatic dependent launch between the library's own kernels (see launch_pdl).
std::atomic<int64_t> opt_bf16_strict{0}, opt_bwd_keep{0}, opt_reserve_sms{0}, opt_pdl{1}, opt_lone_ring{0}, opt_bwd_refill{0}, opt_softmax_two_pass{0}, opt_free_rows{0};
// peer_poll_limit: polls (each sleeping up to 2 us) before a wait on another GPU's counter gives up; process-wide,
// handed to the waiting kernels as an argument at every launch.
// softmax_strict: the softmax / logsumexp forward family with the reference composition's rounding points
// (table-driven exp to 2^-33, fp64 sums, exact division) instead of the approximate exp and fp32 sums.
std::atomic<int64_t> opt_softmax_strict{0};
std::atomic<int64_t> opt_peer_poll_limit{1 << 20};
inline int peer_poll_limit() { return static_cast<int>(opt_peer_poll_limit.load()); }

// ------------------------------------------------------------------ launch planning
struct Plan {
    bool generic = true;
    bool full = false;   // every thread's VPT vectors exist: no bounds checks in the kernel
    int grid = 0, block = 0, smem = 0, vpt = 0, ctas = 0;
    PipeGeom g{};
};

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

enum Which { kFwd = 0, kBwd = 1, kJvp = 2, kSoftmax = 3 };  // kSoftmax: planned like kJvp, never "light"

// Backward variants by elements per thread (= fp64 column sums held in registers): the launch
// bound caps the registers the compiler may use, and with them the threads an SM can hold.
struct BwdVariant {
    int ept, max_threads, regs;
};
constexpr BwdVariant kBwdVariants[3] = {{8, 1024, 64}, {16, 768, 80}, {32, 512, 128}};

// narr: arrays staged per tile; ngamma: [hidden] fp32 vectors kept in shared memory.
// extra_static: statically declared shared memory of the kernel, charged against the per-CTA limit.
void plan_launch(Which which, int64_t rows, int64_t hidden, int elem, int narr, int ngamma, const DevInfo& d,
                 Plan* p, int extra_static = 0, bool heavy = false, int fast = 0) {
    p->generic = true;
    if (opt_force_generic.load() || rows <= 0) return;
    const int64_t row_bytes64 = hidden * elem;
    if (row_bytes64 % 16 != 0 || row_bytes64 > (1 << 20)) return;
    const int row_bytes = static_cast<int>(row_bytes64);
    const int nvec = row_bytes / 16;
    const int epv = 16 / elem;

    // threads per row (G) and vectors per thread (VPT).  Measured on B200: the fixed cost per
    // row and thread (barrier, two reductions, statistics) is large, so MORE elements per thread
    // win: 32 per thread in the backward (the most whose fp64 column sums fit in registers).
    int vpt = 0, G = 0, max_threads = 1024, regs = 64;
    if (which == kBwd && fast) {
        // fp32-accumulating backward (rmsnorm_bwd_fast): 32 elements per thread; fast == 1 keeps x and gy in
        // registers between the passes (launch bound 512 threads), fast == 2 re-reads the tile (768 threads)
        // fast == 3: 64 elements per thread, tile re-read (half the per-row fixed cost per element; 384 threads)
        vpt = (fast == 3 ? 64 : 32) / epv;
        G = round_up((nvec + vpt - 1) / vpt, 32);
        max_threads = fast == 2 ? 768 : (fast == 3 ? 384 : 512);
        regs = fast == 2 ? 80 : (fast == 3 ? 168 : 128);
        if (G > max_threads) return;
    } else if (which == kBwd) {
        const int want = static_cast<int>(opt_ept.load());
        bool found = false;
        for (int pass = 0; pass < 2 && !found; ++pass)
            for (int i = 2; i >= 0 && !found; --i) {
                const BwdVariant& bv = kBwdVariants[i];
                if (pass == 0 && want && bv.ept != want) continue;
                if (bv.ept < epv) continue;
                const int v = bv.ept / epv;
                const int g = round_up((nvec + v - 1) / v, 32);
                if (g > bv.max_threads) continue;
                vpt = v; G = g; max_threads = bv.max_threads; regs = bv.regs;
                found = true;
            }
        if (!found) return;
    } else {
        // the softmax kernels pay two or three reductions per row: 32 elements per thread amortise them
        vpt = (which == kSoftmax && elem == 4) ? 8 : 4;
        G = round_up((nvec + vpt - 1) / vpt, 32);
        if (G > 1024) {
            vpt = 8;
            G = round_up((nvec + vpt - 1) / vpt, 32);
            if (G > 1024) {
                if (which == kFwd) return;
                G = 1024;  // the jvp kernel loops over its vectors
            }
        }
    }
    const int gamma_bytes = static_cast<int>(hidden) * 4;  // always fp32 in shared memory
    const int max_stages = 4;                              // measured: depth beyond 3-4 tiles buys nothing
    auto tile_stride_of = [&](int rpt) { return round_up(rpt * row_bytes, 128); };
    auto stages_for = [&](int rpt, int c) {
        const int nw = rpt * G / 32;
        const int fixed = ngamma * gamma_bytes + 8 * nw * 8 /*reduction scratch*/ + 8 * 16 /*barriers*/ + 32 /*flag, slot counters*/ + 112 /*slack*/ +
                          extra_static;
        int avail = d.smem_per_sm / c - 1024;  // the runtime reserves 1 KB per resident CTA
        if (avail > d.smem_optin) avail = d.smem_optin;
        const int s = (avail - fixed) / (narr * tile_stride_of(rpt));
        return s > max_stages ? max_stages : s;
    };
    // Rows per tile and CTAs per SM: maximise resident threads subject to the ring depth (2 tiles
    // per CTA when several CTAs share the SM, 3 for a lone CTA), the register file and the thread
    // limit; on a tie prefer more, smaller CTAs.  The fp32 RMSNorm forward has so few instructions
    // per byte that 512 threads per SM in one CTA are enough, and measurably better than more (6.5
    // against 5.5 TB/s); its jvp, two arrays wide, is the other way round (5.9 -> 6.6 TB/s).
    int target = static_cast<int>(opt_threads.load());
    if (target <= 0) target = max_threads;
    if (target > max_threads) target = max_threads;
    const int want_ctas = static_cast<int>(opt_ctas_per_sm.load());
    // heavy: the caller's kernel has several times the instructions per byte of the RMSNorm forward (LayerNorm:
    // measured 4.5 -> 5.4-6.4 TB/s in fp32 when it gets the full thread count)
    const bool light = !heavy && which == kFwd && elem == 4;
    // The fp32-accumulating 16-bit forward is as light per byte as the fp32 one, and measured the same way:
    // ONE CTA per SM with about 768 threads streams 6-15 % faster than two or four CTAs on every width tried
    // (8192: 6.25 against 5.70 TB/s, 5120: 6.59 / 5.52, 12288: 6.3-6.7 / 5.88, 1000: 6.07 / 5.36, 4096: 6.25 / 5.49).
    const bool light16 = !heavy && which == kFwd && elem == 2 && narr == 1 && !opt_bf16_strict.load();
    const int max_resident = (light || light16) && !want_ctas && !opt_threads.load() ? (light16 ? 768 : 512) : 2048;
    // The forward with the fused residual add (two arrays in, two out) is an exception, measured on the
    // 32-layer stack shape: ONE CTA per SM streams best -- bf16 with the usual tile (6.4 against 6.2 TB/s),
    // fp32 with a single row group and a two-slot ring (6.45-6.55 against 5.9 TB/s; a third slot brings it
    // back down).
    // (!heavy: the LayerNorm backward also plans as kFwd with two arrays, and one CTA per SM halves it)
    const bool fused_fwd = !heavy && which == kFwd && narr == 2 && !want_ctas && (elem == 2 || G >= 256);
    // The fp32 LayerNorm forward (heavy, one array): two 512-thread CTAs with a two-slot ring beat four
    // 256-thread ones on every fp32 shape measured (6.1-6.2 against 5.25 TB/s at 32768 x 4096, 5.7 against
    // 5.1 at hidden 1024); in bf16, where the kernel is bound by instruction issue, four stay ahead.
    const bool ln_fwd32 = heavy && which == kFwd && narr == 1 && elem == 4;
    // The fp32-accumulating 16-bit LayerNorm forward takes two CTAs per SM as well (65536 rows of bf16, two / four
    // / one CTA: 8192 columns 6.17 / 5.60 / 6.27 TB/s, 4096: 5.94 / 5.76 / 5.61, 5120: 5.93 / 5.68 / 5.58, 12288:
    // 6.31 / no ring / 5.64, 2048: 5.84 / 5.22 / 5.55; only at 1000 columns four stay ahead, 4.70 against 4.55).
    const bool ln_fwd16 = heavy && which == kFwd && narr == 1 && elem == 2 && !opt_bf16_strict.load();
    const int c_hi = want_ctas ? want_ctas : (fused_fwd || light16 ? 1 : (ln_fwd32 || ln_fwd16 ? 2 : 4));
    int rpt = 0, ctas = 0, S = 0, best = 0;
    const int lone_ring = opt_lone_ring.load() == 2 ? 2 : 3;
    for (int c = (want_ctas ? want_ctas : 1); c <= c_hi; ++c)
        for (int r = target / G > 0 ? target / G : 1; r >= 1; --r) {
            if (r > rows && r > 1) continue;
            const int blk = r * G;
            if (blk * c > max_resident && !(c == 1 && r == 1)) continue;
            if (static_cast<int64_t>(regs) * blk * c > 65536) continue;
            const int st = stages_for(r, c);
            if (st < 2 || (c == 1 && st < lone_ring && r > 1)) continue;  // a lone CTA wants a 3-deep ring
            const bool better = blk * c > best || (blk * c == best && !light);
            if (better) { best = blk * c; rpt = r; ctas = c; S = st; }
            break;  // the largest tile that fits for this CTA count
        }
    // (fused-add forward, fp32, wide rows: a single row group and a two-slot ring, see above)
    // (measured again with the fp32-accumulating 16-bit kernel: 8192 6.82 against 5.92 TB/s, 4096 6.64 / 5.87,
    //  12288 6.18 / 5.88; so the rule holds for both element sizes when the strict 16-bit kernel is not asked for)
    if (fused_fwd && (elem == 4 || !opt_bf16_strict.load()) && G >= 256 && !opt_threads.load() && stages_for(1, 1) >= 2) {
        rpt = 1; ctas = 1; S = 2;
    }
    if (rpt == 0) return;
    // The plain forward streams best with a shallow ring (measured: fp32 3 slots against 4: +1.5 %; bf16 with
    // short rows 2 against 3: +4 %): deeper prefetch only scatters the DRAM accesses of an SM over more rows.
    if (which == kFwd && !heavy && narr == 1) {
        const int cap = elem == 4 ? 3 : 2;
        if (S > cap && !(opt_stages.load() > cap)) S = cap;
    }
    if (ln_fwd32 && ctas > 1 && S > 2) S = 2;
    const int want_stages = static_cast<int>(opt_stages.load());
    if (want_stages >= 2 && want_stages < S) S = want_stages;
    const int block = rpt * G;
    const int nwarps = block / 32;
    // Backward with rows that one warp owns (G == 32, hidden <= 32 elements-per-thread): let every warp
    // take several rows of a tile back to back, so the block-wide barrier is paid once per tile, as long
    // as the ring stays three tiles deep.
    int rpw = 1;
    if (which == kBwd && !fast && G == 32 && vpt * epv == 32) {
        const int want_rpw = static_cast<int>(opt_rpw.load());
        for (int cand = (want_rpw > 0 ? want_rpw : 4); cand >= 2; --cand) {
            if (static_cast<int64_t>(rpt) * cand > rows) continue;
            int avail = d.smem_per_sm / ctas - 1024;
            if (avail > d.smem_optin) avail = d.smem_optin;
            const int fixed = ngamma * gamma_bytes + 8 * nwarps * 8 + 8 * 16 + 32 + 112 + extra_static;
            const int st = (avail - fixed) / (narr * tile_stride_of(rpt * cand));
            if (st >= 3 || (want_rpw > 0 && st >= 2)) {
                rpw = cand;
                if (st < S) S = st;
                break;
            }
        }
        if (want_rpw == 1) rpw = 1;
    }
    rpt *= rpw;
    const int tile_stride = tile_stride_of(rpt);
    const int stage_stride = narr * tile_stride;

    PipeGeom& g = p->g;
    g.rows = rows;
    g.hidden = static_cast<int>(hidden);
    g.nvec = nvec;
    g.row_bytes = row_bytes;
    g.rows_per_tile = rpt;
    g.rows_per_warp = rpw;
    g.group_threads = G;
    g.stages = S;
    g.tile_stride = tile_stride;
    g.stage_stride = stage_stride;
    g.ntiles = (rows + rpt - 1) / rpt;
    int off = S * stage_stride;
    g.off_gamma = off;
    off += gamma_bytes * (ngamma > 0 ? 1 : 0);
    g.off_gamma2 = off;
    off += gamma_bytes * (ngamma > 1 ? 1 : 0);
    off = round_up(off, 16);
    g.off_red = off;
    off += 8 * nwarps * 8;
    g.off_bar = off;
    off += 8 * 16;
    g.off_flag = off;
    off += 32;   // the abort flag, then one release counter per ring slot (at most four)
    g.pdl_early = opt_pdl.load() == 2;
    // (the 64-element backward only; "bwd_refill" 1 / 2 force late / early)
    // (the 64-element backward; plan_bwd decides for the 32-element re-reading one; "bwd_refill" 1 / 2 force late / early)
    g.early_refill = fast == 3 && (opt_bwd_refill.load() == 2 || (opt_bwd_refill.load() == 0 && rpt == 1));
    p->smem = off;
    p->block = block;
    p->vpt = vpt;
    p->full = (vpt * G == nvec);
    int reserve = static_cast<int>(opt_reserve_sms.load());
    if (reserve < 0 || reserve >= d.sms) reserve = 0;
    int64_t grid = static_cast<int64_t>(d.sms - reserve) * ctas;
    if (grid > g.ntiles) grid = g.ntiles;
    p->ctas = ctas;
    p->grid = static_cast<int>(grid);
    p->generic = false;
}

// The backward's plan: 16-bit I/O takes the fp32-accumulating kernel (unless "bf16_strict"), which exists with
// three register budgets ("bwd_keep" 1, 2, 3 force one): 64 elements per thread where that fits (see below);
// else, of the two 32-element forms, the one that holds more threads on an SM, and on a tie the
// register-keeping one, which has fewer instructions per element.
void plan_bwd(int64_t rows, int64_t hidden, int elem, int narr, int ngamma, const DevInfo& d, Plan* p, bool* keep) {
    *keep = false;
    if (elem == 2 && !opt_bf16_strict.load()) {
        Plan pk, pn;
        plan_launch(kBwd, rows, hidden, elem, narr, ngamma, d, &pk, 0, false, 1);
        plan_launch(kBwd, rows, hidden, elem, narr, ngamma, d, &pn, 0, false, 2);
        const int64_t want_keep = opt_bwd_keep.load();
        // 64 elements per thread halve the fixed cost per row and thread (barrier, two reductions): measured
        // +10 % at 4096 columns, +2 % at 8192, but -8 % at 12288, where a row group of 192 threads is all an SM
        // can hold.  Taken when every thread's vectors exist, a row is at most 16 KB and 256 threads stay resident.
        if (want_keep == 3 || want_keep == 0 || want_keep == 4) {
            Plan pw;
            plan_launch(kBwd, rows, hidden, elem, narr, ngamma, d, &pw, 0, false, 3);
            const bool fits = !pw.generic && pw.full;
            if (fits && (want_keep >= 3 || (hidden * elem <= 16384 && pw.block * pw.ctas >= 256))) { *p = pw; return; }
        }
        if (want_keep == 1) *keep = !pk.generic;
        else if (want_keep == 2) *keep = pn.generic && !pk.generic;
        // (rows that one warp owns, hidden <= 1024: the register-keeping form measured 4-5 % ahead at 1000 columns)
        else *keep = !pk.generic && (pn.generic || pk.block * pk.ctas >= pn.block * pn.ctas || pk.g.group_threads == 32);
        // The re-reading form with the early slot refill (instantiated for up to 640 resident threads, full tilings,
        // gamma): measured settled, 65536 rows -- 5120 columns (two rows per tile) 557 against 575 us per step;
        // 12288 and 10240 columns (one CTA per SM, one row per tile) 1367 / 1197 against 1382 / 1226 us with the
        // register-keeping form, which it therefore replaces there; at 7168 columns (two CTAs) the register-keeping
        // form stays ahead (803 against 824 us), and with three or more rows per tile the early refill loses.
        const int64_t refill = opt_bwd_refill.load();
        const bool early_ok = refill != 1 && ngamma == 1 && !pn.generic && pn.full && pn.g.rows_per_tile <= 2 &&
                              pn.block * pn.ctas <= 640;
        if (*keep && want_keep == 0 && early_ok && pn.ctas == 1 && pn.g.rows_per_tile == 1) *keep = false;
        *p = *keep ? pk : pn;
        if (!*keep) p->g.early_refill = early_ok;
        return;
    }
    plan_launch(kBwd, rows, hidden, elem, narr, ngamma, d, p);
}

// Launch of a kernel that begins with pdl_wait(): with the "pdl" option (default on) it carries the
// programmatic-stream-serialization attribute, so its CTAs are placed while the kernel before it in the
// stream drains and the gap between dependent kernels shrinks to the wait itself.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = opt_pdl.load() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename K>
int set_smem(K kernel, int bytes) {
    // Raising the limit is idempotent and cheap; doing it on every call keeps this correct for
    // every device and context without a cache.
    AGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return AGB_OK;
}

int check_common(int64_t rows, int64_t hidden, int dtype) {
    if (rows < 0 || hidden <= 0) return fail(AGB_ERR_INVALID_ARG, "rows=%lld hidden=%lld", (long long)rows, (long long)hidden);
    if (dtype != AGB_F32 && dtype != AGB_BF16) return fail(AGB_ERR_UNSUPPORTED, "dtype %d (only AGB_F32, AGB_BF16)", dtype);
    if (hidden > (1LL << 30)) return fail(AGB_ERR_UNSUPPORTED, "hidden %lld too large", (long long)hidden);
    return AGB_OK;
}
int check_ptr(const void* p, const char* name, int elem, bool required = true) {
    if (!p) return required ? fail(AGB_ERR_INVALID_ARG, "%s is NULL", name) : AGB_OK;
    if (reinterpret_cast<uintptr_t>(p) % elem) return fail(AGB_ERR_MISALIGNED, "%s not aligned to %d bytes", name, elem);
    return AGB_OK;
}
#define AGB_TRY(expr)                 \
    do {                              \
        int s__ = (expr);             \
        if (s__ != AGB_OK) return s__; \
    } while (0)

inline int generic_grid(int64_t rows, const DevInfo& d) {
    int64_t g = static_cast<int64_t>(d.sms) * 8;
    return static_cast<int>(rows < g ? rows : g);
}
// dgamma partial rows ([hidden] fp64 each, one per CTA of the backward): a caller workspace must hold at
// least max_partials() rows; the staged backward may run up to kMaxCtasPerSm CTAs per SM and is given as
// many of them as the workspace has rows for (agb_rmsnorm_bwd_workspace_bytes() asks for all of them).
constexpr int kMaxCtasPerSm = 4;
inline int max_partials(const DevInfo& d) { return 2 * d.sms; }

// ------------------------------------------------------------------ typed launchers
template <typename T>
int launch_fwd(const void* x, const void* r, const void* gamma, void* h, void* y, float* rstd, int64_t rows,
               int64_t hidden, float eps, bool fuse, cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    const bool al = aligned16(x) && aligned16(y) && (!fuse || (aligned16(r) && aligned16(h))) && (!gamma || aligned16(gamma));
    if (al) plan_launch(kFwd, rows, hidden, sizeof(T), fuse ? 2 : 1, gamma ? 1 : 0, *d, &p);
    if (p.generic) {
        const int grid = generic_grid(rows, *d);
        if (fuse)
            agb::rmsnorm_fwd_generic<T, true><<<grid, agb::kGenericThreads, 0, st>>>(
                (const T*)x, (const T*)r, (const T*)gamma, (T*)h, (T*)y, rstd, rows, (int)hidden, eps);
        else
            agb::rmsnorm_fwd_generic<T, false><<<grid, agb::kGenericThreads, 0, st>>>(
                (const T*)x, nullptr, (const T*)gamma, nullptr, (T*)y, rstd, rows, (int)hidden, eps);
        return after_launch("rmsnorm_fwd_generic");
    }
    agb::FwdArgs a{p.g, x, r, gamma, h, y, rstd, eps};
    if constexpr (sizeof(T) == 2) if (!opt_bf16_strict.load()) {
        const float hinv = 1.0f / static_cast<float>(hidden);
#define AGB_LAUNCH_FWDF_R(V, HG, FA, FU, FR)                                                 \
    do {                                                                                     \
        AGB_TRY(set_smem(agb::rmsnorm_fwd_fast<T, V, HG, FA, FU, FR>, p.smem));              \
        AGB_CUDA(launch_pdl(agb::rmsnorm_fwd_fast<T, V, HG, FA, FU, FR>, p.grid, p.block, p.smem, st, a, hinv)); \
    } while (0)
#define AGB_LAUNCH_FWDF(V, HG, FA, FU) AGB_LAUNCH_FWDF_R(V, HG, FA, FU, false)
#define AGB_FWDF_BY_FLAGS(V, FU)                                 \
    do {                                                         \
        if (gamma && fuse) AGB_LAUNCH_FWDF(V, true, true, FU);   \
        else if (gamma) AGB_LAUNCH_FWDF(V, true, false, FU);     \
        else if (fuse) AGB_LAUNCH_FWDF(V, false, true, FU);      \
        else AGB_LAUNCH_FWDF(V, false, false, FU);               \
    } while (0)
        // rows that one warp owns, several per tile, gamma, no fused add: the form without a block-wide barrier
        // (measured 65536 x 1000 bf16: 6143 against 5923 GB/s; 262144 x 512: 5574 against 5237; level at 768 / 1024)
        const bool free_rows = p.g.group_threads == 32 && p.block > 32 && gamma && !fuse && p.vpt == 4 &&
                               opt_free_rows.load() != 1;
        if (free_rows && p.full) AGB_LAUNCH_FWDF_R(4, true, false, true, true);
        else if (free_rows) AGB_LAUNCH_FWDF_R(4, true, false, false, true);
        else if (p.vpt == 4 && p.full) AGB_FWDF_BY_FLAGS(4, true);
        else if (p.vpt == 4) AGB_FWDF_BY_FLAGS(4, false);
        else AGB_FWDF_BY_FLAGS(8, false);
#undef AGB_FWDF_BY_FLAGS
#undef AGB_LAUNCH_FWDF
#undef AGB_LAUNCH_FWDF_R
        return after_launch("rmsnorm_fwd_fast");
    }
#define AGB_LAUNCH_FWD(V, HG, FA, FU)                                                   \
    do {                                                                                \
        AGB_TRY(set_smem(agb::rmsnorm_fwd_staged<T, V, HG, FA, FU>, p.smem));           \
        AGB_CUDA(launch_pdl(agb::rmsnorm_fwd_staged<T, V, HG, FA, FU>, p.grid, p.block, p.smem, st, a)); \
    } while (0)
#define AGB_FWD_BY_FLAGS(V, FU)                          \
    do {                                                 \
        if (gamma && fuse) AGB_LAUNCH_FWD(V, true, true, FU);   \
        else if (gamma) AGB_LAUNCH_FWD(V, true, false, FU);     \
        else if (fuse) AGB_LAUNCH_FWD(V, false, true, FU);      \
        else AGB_LAUNCH_FWD(V, false, false, FU);               \
    } while (0)
    if (p.vpt == 4 && p.full) AGB_FWD_BY_FLAGS(4, true);
    else if (p.vpt == 4) AGB_FWD_BY_FLAGS(4, false);
    else AGB_FWD_BY_FLAGS(8, false);
#undef AGB_FWD_BY_FLAGS
#undef AGB_LAUNCH_FWD
    return after_launch("rmsnorm_fwd_staged");
}

// Set by agb_peer_rmsnorm_bwd around its own call of the backward (same thread, same call stack): the
// column reduction of that call then waits for the peers' acknowledgements and publishes the sums itself.
thread_local const agb::PeerHook* t_reduce_hook = nullptr;
thread_local bool t_reduce_hook_used = false;

int launch_dgamma_reduce(const double* partials, int P, int64_t hidden, void* dgamma, int dgamma_dtype,
                         int accumulate, cudaStream_t st, bool behind_backward = true) {
    const int mode = dgamma_dtype == AGB_F64 ? (accumulate ? 3 : 2) : (accumulate ? 1 : 0);
    dim3 block(agb::kReduceCols, agb::kReduceLanes);
    const int grid = static_cast<int>((hidden + agb::kReduceCols - 1) / agb::kReduceCols);
    if (t_reduce_hook && mode == 2) {
        agb::dgamma_reduce_publish_kernel<<<grid, block, 0, st>>>(partials, P, (int)hidden, *t_reduce_hook);
        t_reduce_hook_used = true;
        return after_launch("dgamma_reduce_publish");
    }
    // placed early only when the kernel before it in this stream is the backward that wrote the partials
    if (behind_backward) AGB_CUDA(launch_pdl(agb::dgamma_reduce_kernel, grid, block, 0, st, partials, P, (int)hidden, dgamma, mode));
    else agb::dgamma_reduce_kernel<<<grid, block, 0, st>>>(partials, P, (int)hidden, dgamma, mode);
    return after_launch("dgamma_reduce");
}

template <typename T>
int launch_bwd(const void* x, const void* gamma, const float* rstd, const void* gy, const void* dx_add, void* dx,
               void* dgamma, int dgamma_dtype, int accumulate_dgamma, void* workspace, size_t workspace_bytes,
               int64_t rows, int64_t hidden, cudaStream_t st, int* partials_only = nullptr) {
    // partials_only: leave the partial rows in the workspace, report their number, run no reduction
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    const bool want_dg = gamma != nullptr && (dgamma != nullptr || partials_only != nullptr);
    if (partials_only) *partials_only = 0;
    if (want_dg) {
        const size_t need = static_cast<size_t>(max_partials(*d)) * hidden * sizeof(double);
        if (!workspace || workspace_bytes < need)
            return fail(AGB_ERR_WORKSPACE, "workspace %zu bytes, need %zu", workspace_bytes, need);
        if (reinterpret_cast<uintptr_t>(workspace) % 16) return fail(AGB_ERR_MISALIGNED, "workspace not 16-byte aligned");
    }
    if (rows == 0) {
        if (want_dg && !accumulate_dgamma && !partials_only)
            AGB_CUDA(cudaMemsetAsync(dgamma, 0, hidden * (dgamma_dtype == AGB_F64 ? 8 : 4), st));
        return AGB_OK;
    }
    int add_mode = 0;
    if (dx_add) add_mode = (dx_add == gy) ? 2 : 1;
    Plan p;
    const bool al = aligned16(x) && aligned16(gy) && aligned16(dx) && (!gamma || aligned16(gamma)) &&
                    (add_mode != 1 || aligned16(dx_add));
    const bool fast = sizeof(T) == 2 && !opt_bf16_strict.load();
    bool keep = false;
    if (al) plan_bwd(rows, hidden, sizeof(T), add_mode == 1 ? 3 : 2, gamma ? 1 : 0, *d, &p, &keep);
    if (want_dg && !p.generic) {
        // every CTA writes the partial row of its block index: never launch more CTAs than the workspace has rows
        const size_t cap = workspace_bytes / (static_cast<size_t>(hidden) * sizeof(double));
        if (static_cast<size_t>(p.grid) > cap) p.grid = static_cast<int>(cap);
    }
    double* partials = static_cast<double*>(workspace);
    int P = 0;
    if (p.generic) {
        if (want_dg) {
            // column sums first: dx may alias an input of theirs only through dx_add, never x or gy
            P = static_cast<int>(rows < max_partials(*d) ? rows : max_partials(*d));
            const int64_t rpc = (rows + P - 1) / P;
            P = static_cast<int>((rows + rpc - 1) / rpc);
            dim3 grid((unsigned)((hidden + agb::kGenericThreads - 1) / agb::kGenericThreads), (unsigned)P);
            agb::dgamma_generic_partial<T><<<grid, agb::kGenericThreads, 0, st>>>((const T*)x, (const T*)gy, rstd,
                                                                                 partials, rows, (int)hidden, rpc);
            AGB_TRY(after_launch("dgamma_generic_partial"));
        }
        const float hf = static_cast<float>(hidden);
        agb::rmsnorm_bwd_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)x, (const T*)gamma, rstd, (const T*)gy, (const T*)dx_add, (T*)dx, rows, (int)hidden, hf, 1.0f / hf);
        AGB_TRY(after_launch("rmsnorm_bwd_generic"));
    } else if (fast) {
      if constexpr (sizeof(T) == 2) {
        const float hf = static_cast<float>(hidden);
        agb::BwdArgs a{p.g, x, gy, dx_add, gamma, rstd, dx, want_dg ? partials : nullptr, add_mode, hf, 1.0f / hf};
        P = p.grid;
        constexpr int kV = 32 / (16 / static_cast<int>(sizeof(T)));
#define AGB_LAUNCH_FAST_V(V, HG, FU, MT, KP, EA)                                              \
    do {                                                                                      \
        AGB_TRY(set_smem(agb::rmsnorm_bwd_fast<T, V, HG, FU, MT, KP, EA>, p.smem));           \
        AGB_CUDA(launch_pdl(agb::rmsnorm_bwd_fast<T, V, HG, FU, MT, KP, EA>, p.grid, p.block, p.smem, st, a)); \
    } while (0)
#define AGB_LAUNCH_FAST(HG, FU, MT, KP) AGB_LAUNCH_FAST_V(kV, HG, FU, MT, KP, 0)
#define AGB_FAST_BY_FLAGS(MT, KP)                                  \
    do {                                                           \
        if (gamma && p.full) AGB_LAUNCH_FAST(true, true, MT, KP);  \
        else if (gamma) AGB_LAUNCH_FAST(true, false, MT, KP);      \
        else if (p.full) AGB_LAUNCH_FAST(false, true, MT, KP);     \
        else AGB_LAUNCH_FAST(false, false, MT, KP);                \
    } while (0)
        if (p.vpt == 2 * kV) {   // 64 elements per thread (planned only when full)
            // With at most 256 resident threads per SM a thread may use 255 registers: x (unpacked) and gy (as loaded)
            // stay in registers between the passes as well (224 registers), so pass 2 reads only gamma from shared
            // memory and unpacks only gy.  Measured settled at 65536 x 8192 bf16: step 855.5 against 881.6 us, the
            // backward alone 508.6 against 533.7 us.  "bwd_keep" 3 forces the re-reading form, 4 this one.
            if (gamma && p.g.early_refill && opt_bwd_keep.load() != 3 && p.block * p.ctas <= 256)
                AGB_LAUNCH_FAST_V(2 * kV, true, true, 256, true, 1);
            else if (gamma && p.g.early_refill) AGB_LAUNCH_FAST_V(2 * kV, true, true, 384, false, 1);
            else if (gamma) AGB_LAUNCH_FAST_V(2 * kV, true, true, 384, false, 0);
            else AGB_LAUNCH_FAST_V(2 * kV, false, true, 384, false, 0);
        } else if (!keep && gamma && p.full && p.g.early_refill && p.block * p.ctas <= 384) {
            AGB_LAUNCH_FAST_V(kV, true, true, 384, false, 1);
        } else if (!keep && gamma && p.full && p.g.early_refill && p.block * p.ctas <= 640) {
            AGB_LAUNCH_FAST_V(kV, true, true, 640, false, 1);
        } else if (keep) AGB_FAST_BY_FLAGS(512, true);
        else AGB_FAST_BY_FLAGS(768, false);
#undef AGB_LAUNCH_FAST_V
#undef AGB_FAST_BY_FLAGS
#undef AGB_LAUNCH_FAST
        AGB_TRY(after_launch("rmsnorm_bwd_fast"));
      }
    } else {
        const float hf = static_cast<float>(hidden);
        agb::BwdArgs a{p.g, x, gy, dx_add, gamma, rstd, dx, want_dg ? partials : nullptr, add_mode, hf, 1.0f / hf};
        P = p.grid;
#define AGB_LAUNCH_BWD2(V, HG, FU, MT, P2)                                                   \
    do {                                                                                     \
        AGB_TRY(set_smem(agb::rmsnorm_bwd_staged<T, V, HG, FU, MT, P2>, p.smem));            \
        AGB_CUDA(launch_pdl(agb::rmsnorm_bwd_staged<T, V, HG, FU, MT, P2>, p.grid, p.block, p.smem, st, a)); \
    } while (0)
#define AGB_LAUNCH_BWD(V, HG, FU, MT)                     \
    do {                                                  \
        if (pow2) AGB_LAUNCH_BWD2(V, HG, FU, MT, true);   \
        else AGB_LAUNCH_BWD2(V, HG, FU, MT, false);       \
    } while (0)
        const bool pow2 = (hidden & (hidden - 1)) == 0;
#define AGB_BWD_BY_FLAGS(V, MT)                                  \
    do {                                                         \
        if (gamma && p.full) AGB_LAUNCH_BWD(V, true, true, MT);  \
        else if (gamma) AGB_LAUNCH_BWD(V, true, false, MT);      \
        else if (p.full) AGB_LAUNCH_BWD(V, false, true, MT);     \
        else AGB_LAUNCH_BWD(V, false, false, MT);                \
    } while (0)
        // elements per thread 8 / 16 / 32  <->  launch bound 1024 / 768 / 512 threads
        constexpr int kEpv = 16 / static_cast<int>(sizeof(T));
        const int ept = p.vpt * kEpv;
        if (p.g.rows_per_warp > 1) {
            // rows-per-warp form (planned only for 32 elements per thread and one-warp rows)
#define AGB_LAUNCH_MULTI(HG, FU, P2)                                                                              \
    do {                                                                                                          \
        AGB_TRY(set_smem(agb::rmsnorm_bwd_staged<T, 32 / kEpv, HG, FU, 512, P2, true>, p.smem));                  \
        AGB_CUDA(launch_pdl(agb::rmsnorm_bwd_staged<T, 32 / kEpv, HG, FU, 512, P2, true>, p.grid, p.block, p.smem, st, a)); \
    } while (0)
#define AGB_MULTI_P2(HG, FU)                        \
    do {                                            \
        if (pow2) AGB_LAUNCH_MULTI(HG, FU, true);   \
        else AGB_LAUNCH_MULTI(HG, FU, false);       \
    } while (0)
            if (gamma && p.full) AGB_MULTI_P2(true, true);
            else if (gamma) AGB_MULTI_P2(true, false);
            else if (p.full) AGB_MULTI_P2(false, true);
            else AGB_MULTI_P2(false, false);
#undef AGB_MULTI_P2
#undef AGB_LAUNCH_MULTI
        } else if (ept == 8) AGB_BWD_BY_FLAGS(8 / kEpv, 1024);
        else if (ept == 16) AGB_BWD_BY_FLAGS(16 / kEpv, 768);
        else AGB_BWD_BY_FLAGS(32 / kEpv, 512);
#undef AGB_BWD_BY_FLAGS
#undef AGB_LAUNCH_BWD
#undef AGB_LAUNCH_BWD2
        AGB_TRY(after_launch("rmsnorm_bwd_staged"));
    }
    if (partials_only) {
        *partials_only = P;
        return AGB_OK;
    }
    if (want_dg) AGB_TRY(launch_dgamma_reduce(partials, P, hidden, dgamma, dgamma_dtype, accumulate_dgamma, st));
    return AGB_OK;
}

template <typename T>
int launch_jvp(const void* x, const void* gamma, const float* rstd, const void* tx, const void* tgamma, void* ty,
               int64_t rows, int64_t hidden, cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    const bool al = aligned16(x) && aligned16(tx) && aligned16(ty) && (!gamma || aligned16(gamma)) &&
                    (!tgamma || aligned16(tgamma));
    if (al) plan_launch(kJvp, rows, hidden, sizeof(T), 2, (gamma ? 1 : 0) + (tgamma ? 1 : 0), *d, &p);
    const float hf = static_cast<float>(hidden);
    if (p.generic) {
        agb::rmsnorm_jvp_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)x, (const T*)gamma, rstd, (const T*)tx, (const T*)tgamma, (T*)ty, rows, (int)hidden, hf);
        return after_launch("rmsnorm_jvp_generic");
    }
    agb::JvpArgs a{p.g, x, tx, gamma, tgamma, rstd, ty, hf};
    if constexpr (sizeof(T) == 2) if (!opt_bf16_strict.load()) {   // 16-bit I/O: fp32 accumulation
        AGB_TRY(set_smem(agb::rmsnorm_jvp_staged<T, true>, p.smem));
        agb::rmsnorm_jvp_staged<T, true><<<p.grid, p.block, p.smem, st>>>(a);
        return after_launch("rmsnorm_jvp_staged");
    }
    AGB_TRY(set_smem(agb::rmsnorm_jvp_staged<T>, p.smem));
    agb::rmsnorm_jvp_staged<T><<<p.grid, p.block, p.smem, st>>>(a);
    return after_launch("rmsnorm_jvp_staged");
}

template <typename T>
int launch_ln_jvp(const void* y, const void* t, const float* var, void* ty, int64_t rows, int64_t hidden, float eps,
                  cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    if (aligned16(y) && aligned16(t) && aligned16(ty)) plan_launch(kJvp, rows, hidden, sizeof(T), 2, 0, *d, &p, 0, true);
    if (p.generic) {
        agb::layernorm_jvp_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)y, (const T*)t, var, (T*)ty, rows, (int)hidden, eps);
        return after_launch("layernorm_jvp_generic");
    }
    agb::LnJvpArgs a{p.g, y, t, var, ty, eps};
    if constexpr (sizeof(T) == 2) if (!opt_bf16_strict.load()) {   // 16-bit I/O: fp32 accumulation
        AGB_TRY(set_smem(agb::layernorm_jvp_staged<T, true>, p.smem));
        agb::layernorm_jvp_staged<T, true><<<p.grid, p.block, p.smem, st>>>(a);
        return after_launch("layernorm_jvp_staged");
    }
    AGB_TRY(set_smem(agb::layernorm_jvp_staged<T>, p.smem));
    agb::layernorm_jvp_staged<T><<<p.grid, p.block, p.smem, st>>>(a);
    return after_launch("layernorm_jvp_staged");
}

// mode: the MODE of softmax_fwd_staged / softmax_fwd_generic.
template <typename T>
int launch_softmax_fwd(int mode, const void* z, const void* t, const void* rowscale, const void* add, void* out,
                       void* out_row, int64_t rows, int64_t hidden, cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    const bool al = aligned16(z) && (!t || aligned16(t)) && (!out || aligned16(out)) && (!add || aligned16(add));
    // arrays per stage: z [, t] [, fp32 scratch = two bf16 row-widths]; fp32 parks e in place over z.
    // The approximate form keeps e in registers (32 values per thread) when the plan gives every thread at most
    // that many, and then needs no scratch at all.
    constexpr int kKeepVecs = 32 / (16 / static_cast<int>(sizeof(T)));   // 8 fp32 vectors, 4 bf16 vectors
    const bool fastmode = !opt_softmax_strict.load();
    bool keep_regs = false;
    if (al && fastmode) {
        plan_launch(kSoftmax, rows, hidden, sizeof(T), mode == 3 ? 2 : 1, 0, *d, &p, agb::kExpTableSize * 8 + agb::kExp32Size * 8);
        keep_regs = !p.generic && static_cast<int64_t>(kKeepVecs) * p.g.group_threads >= p.g.nvec;
    }
    // One pass (softmax_fwd_online) or two: logsumexp and the 16-bit softmax gain everywhere measured (logsumexp
    // +3 to +44 %, bf16 softmax +1 to +16 %); the fp32 softmax gains with wide row groups (16384 columns: 6.17
    // against 5.50 TB/s) and loses with narrow ones (4096 columns, 128 threads per row: 5.37 against 5.94).
    // "softmax_two_pass" 1 / 2 force two / one.
    const int64_t two_pass = opt_softmax_two_pass.load();
    const bool online = keep_regs && mode <= 1 && two_pass != 1 &&
                        (two_pass == 2 || mode == 1 || sizeof(T) == 2 || p.g.group_threads >= 256);
    if (mode == 1 && !online) keep_regs = false;   // (the two-pass logsumexp keeps nothing between its passes)
    const bool scratch = mode != 1 && sizeof(T) == 2 && !keep_regs;
    const int narr = (mode == 3 ? 2 : 1) + (scratch ? 2 : 0);
    if (al && !keep_regs) {
        p = Plan();
        plan_launch(kSoftmax, rows, hidden, sizeof(T), narr, 0, *d, &p, agb::kExpTableSize * 8 + agb::kExp32Size * 8);
    }
    if (p.generic && al && (hidden * static_cast<int64_t>(sizeof(T))) % 16 == 0 && !opt_force_generic.load()) {
        // too wide for the ring, but vectorisable: one 1024-thread CTA per row
        agb::SoftmaxArgs a{};
        a.g.rows = rows; a.g.hidden = static_cast<int>(hidden); a.g.row_bytes = static_cast<int>(hidden * sizeof(T));
        a.g.nvec = a.g.row_bytes / 16;
        a.z = z; a.t = t; a.rowscale = rowscale; a.add = add; a.out = out; a.out_row = out_row;
        const int grid = static_cast<int>(rows < d->sms ? rows : d->sms);   // one 1024-thread CTA per SM
#define AGB_SM_WIDE(M) agb::softmax_fwd_wide<T, M><<<grid, agb::kWideThreads, 0, st>>>(a)
        if (mode == 0) AGB_SM_WIDE(0);
        else if (mode == 1) AGB_SM_WIDE(1);
        else if (mode == 2) AGB_SM_WIDE(2);
        else AGB_SM_WIDE(3);
#undef AGB_SM_WIDE
        return after_launch("softmax_fwd_wide");
    }
    if (p.generic) {
        const int grid = generic_grid(rows, *d);
#define AGB_SM_GENERIC(M)                                                                                         \
    agb::softmax_fwd_generic<T, M><<<grid, agb::kGenericThreads, 0, st>>>((const T*)z, (const T*)t, (const T*)rowscale, \
                                                                         (const T*)add, (T*)out, (T*)out_row, rows, (int)hidden)
        if (mode == 0) AGB_SM_GENERIC(0);
        else if (mode == 1) AGB_SM_GENERIC(1);
        else if (mode == 2) AGB_SM_GENERIC(2);
        else AGB_SM_GENERIC(3);
#undef AGB_SM_GENERIC
        return after_launch("softmax_fwd_generic");
    }
    agb::SoftmaxArgs a{p.g, z, t, rowscale, add, out, out_row, scratch ? (mode == 3 ? 2 : 1) * p.g.tile_stride : 0};
    // softmax and logsumexp forward, approximate arithmetic, row in registers: the one-pass kernel
    if (online) {
        if (mode == 0) {
            AGB_TRY(set_smem(agb::softmax_fwd_online<T, 0, kKeepVecs>, p.smem));
            agb::softmax_fwd_online<T, 0, kKeepVecs><<<p.grid, p.block, p.smem, st>>>(a);
        } else {
            AGB_TRY(set_smem(agb::softmax_fwd_online<T, 1, kKeepVecs>, p.smem));
            agb::softmax_fwd_online<T, 1, kKeepVecs><<<p.grid, p.block, p.smem, st>>>(a);
        }
        return after_launch("softmax_fwd_online");
    }
#define AGB_SM_STAGED(M)                                                              \
    do {                                                                              \
        if (opt_softmax_strict.load()) {                                              \
            AGB_TRY(set_smem(agb::softmax_fwd_staged<T, M, false>, p.smem));          \
            agb::softmax_fwd_staged<T, M, false><<<p.grid, p.block, p.smem, st>>>(a); \
        } else if (keep_regs) {                                                       \
            AGB_TRY(set_smem(agb::softmax_fwd_staged<T, M, true, kKeepVecs>, p.smem));          \
            agb::softmax_fwd_staged<T, M, true, kKeepVecs><<<p.grid, p.block, p.smem, st>>>(a); \
        } else {                                                                      \
            AGB_TRY(set_smem(agb::softmax_fwd_staged<T, M, true>, p.smem));           \
            agb::softmax_fwd_staged<T, M, true><<<p.grid, p.block, p.smem, st>>>(a);  \
        }                                                                             \
    } while (0)
    if (mode == 0) AGB_SM_STAGED(0);
    else if (mode == 1) AGB_SM_STAGED(1);
    else if (mode == 2) AGB_SM_STAGED(2);
    else AGB_SM_STAGED(3);
#undef AGB_SM_STAGED
    return after_launch("softmax_fwd_staged");
}

template <typename T>
int launch_softmax_bwd(const void* y, const void* g, const void* add, void* out, int64_t rows, int64_t hidden,
                       cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    if (aligned16(y) && aligned16(g) && aligned16(out) && (!add || aligned16(add)))
        plan_launch(kSoftmax, rows, hidden, sizeof(T), 2, 0, *d, &p);
    const bool al = aligned16(y) && aligned16(g) && aligned16(out) && (!add || aligned16(add));
    if (p.generic && al && (hidden * static_cast<int64_t>(sizeof(T))) % 16 == 0 && !opt_force_generic.load()) {
        agb::SoftmaxBwdArgs a{};
        a.g.rows = rows; a.g.hidden = static_cast<int>(hidden); a.g.row_bytes = static_cast<int>(hidden * sizeof(T));
        a.g.nvec = a.g.row_bytes / 16;
        a.y = y; a.gr = g; a.add = add; a.out = out;
        const int grid = static_cast<int>(rows < d->sms ? rows : d->sms);
        agb::softmax_bwd_wide<T><<<grid, agb::kWideThreads, 0, st>>>(a);
        return after_launch("softmax_bwd_wide");
    }
    if (p.generic) {
        agb::softmax_bwd_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)y, (const T*)g, (const T*)add, (T*)out, rows, (int)hidden);
        return after_launch("softmax_bwd_generic");
    }
    agb::SoftmaxBwdArgs a{p.g, y, g, add, out};
    AGB_TRY(set_smem(agb::softmax_bwd_staged<T>, p.smem));
    agb::softmax_bwd_staged<T><<<p.grid, p.block, p.smem, st>>>(a);
    return after_launch("softmax_bwd_staged");
}

template <typename T>
int launch_ln_fwd(const void* x, void* y, float* mean, float* var, int64_t rows, int64_t hidden, float eps,
                  cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    if (aligned16(x) && aligned16(y)) plan_launch(kFwd, rows, hidden, sizeof(T), 1, 0, *d, &p, 0, true);
    if (p.generic) {
        agb::layernorm_fwd_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)x, (T*)y, mean, var, rows, (int)hidden, eps);
        return after_launch("layernorm_fwd_generic");
    }
    agb::LnFwdArgs a{p.g, x, y, mean, var, eps};
#define AGB_LN_FWD(V, FU)                                                                    \
    do {                                                                                     \
        if (sizeof(T) == 2 && !opt_bf16_strict.load()) {                                     \
            AGB_TRY(set_smem(agb::layernorm_fwd_staged<T, V, FU, true>, p.smem));            \
            agb::layernorm_fwd_staged<T, V, FU, true><<<p.grid, p.block, p.smem, st>>>(a);   \
        } else {                                                                             \
            AGB_TRY(set_smem(agb::layernorm_fwd_staged<T, V, FU, false>, p.smem));           \
            agb::layernorm_fwd_staged<T, V, FU, false><<<p.grid, p.block, p.smem, st>>>(a);  \
        }                                                                                    \
    } while (0)
    if (p.vpt == 4 && p.full) AGB_LN_FWD(4, true);
    else if (p.vpt == 4) AGB_LN_FWD(4, false);
    else AGB_LN_FWD(8, false);
#undef AGB_LN_FWD
    return after_launch("layernorm_fwd_staged");
}

template <typename T>
int launch_ln_bwd(const void* x, const float* mean, const float* var, const void* gy, const void* dx_add, void* dx,
                  int64_t rows, int64_t hidden, float eps, cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    int add_mode = 0;
    if (dx_add) add_mode = (dx_add == gy) ? 2 : 1;
    Plan p;
    if (aligned16(x) && aligned16(gy) && aligned16(dx) && (add_mode != 1 || aligned16(dx_add)))
        plan_launch(kFwd, rows, hidden, sizeof(T), add_mode == 1 ? 3 : 2, 0, *d, &p, 0, true);
    const float hf = static_cast<float>(hidden);
    if (p.generic) {
        agb::layernorm_bwd_generic<T><<<generic_grid(rows, *d), agb::kGenericThreads, 0, st>>>(
            (const T*)x, mean, var, (const T*)gy, (const T*)dx_add, (T*)dx, rows, (int)hidden, eps, hf, 2.0f / hf);
        return after_launch("layernorm_bwd_generic");
    }
    agb::LnBwdArgs a{p.g, x, gy, dx_add, mean, var, dx, add_mode, eps, hf, 2.0f / hf};
#define AGB_LN_BWD(V, FU)                                                                    \
    do {                                                                                     \
        if (sizeof(T) == 2 && !opt_bf16_strict.load()) {                                     \
            AGB_TRY(set_smem(agb::layernorm_bwd_staged<T, V, FU, true>, p.smem));            \
            agb::layernorm_bwd_staged<T, V, FU, true><<<p.grid, p.block, p.smem, st>>>(a);   \
        } else {                                                                             \
            AGB_TRY(set_smem(agb::layernorm_bwd_staged<T, V, FU, false>, p.smem));           \
            agb::layernorm_bwd_staged<T, V, FU, false><<<p.grid, p.block, p.smem, st>>>(a);  \
        }                                                                                    \
    } while (0)
    if (p.vpt == 4 && p.full) AGB_LN_BWD(4, true);
    else if (p.vpt == 4) AGB_LN_BWD(4, false);
    else AGB_LN_BWD(8, false);
#undef AGB_LN_BWD
    return after_launch("layernorm_bwd_staged");
}

inline int ew_grid(int64_t work_items, const DevInfo& d) {
    int64_t g = (work_items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(d.sms) * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}


// ------------------------------------------------------------------ built-in scratch (agb_rmsnorm_bwd_static)
// The partial dgamma rows of agb_rmsnorm_bwd_static live in this array instead of a caller
// workspace.  Every device that loads the library carries it until the process exits.
// In host code the name below is only a handle for the runtime, NOT a device address: the
// address is asked for once per device (with that device current) and cached.
constexpr size_t kStaticScratchBytes = AGB_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_scratch_mu;

int static_scratch_for_current_device(void** out) {
    int dev = 0;
    AGB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(AGB_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_scratch_mu);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        AGB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (p == nullptr) return fail(AGB_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_static_scratch_addr[dev] = p;
    }
    *out = g_static_scratch_addr[dev];
    return AGB_OK;
}

}  // namespace

// ====================================================================== C ABI
extern "C" {

int agb_version(void) { return 100; }

const char* agb_status_string(int s) {
    switch (s) {
        case AGB_OK: return "ok";
        case AGB_ERR_INVALID_ARG: return "invalid argument";
        case AGB_ERR_UNSUPPORTED: return "unsupported dtype or shape";
        case AGB_ERR_MISALIGNED: return "misaligned pointer";
        case AGB_ERR_CUDA: return "CUDA error";
        case AGB_ERR_WORKSPACE: return "workspace missing or too small";
        case AGB_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}
const char* agb_last_error(void) { return t_err; }
uint64_t agb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int agb_device_status(void) {
    int v = 0, zero = 0;
    AGB_CUDA(cudaDeviceSynchronize());
    AGB_CUDA(cudaMemcpyFromSymbol(&v, agb::g_device_status, sizeof(int)));
    if (v != 0) AGB_CUDA(cudaMemcpyToSymbol(agb::g_device_status, &zero, sizeof(int)));
    if (v != 0) return fail(v, "a kernel's bounded shared-memory wait ran out");
    return AGB_OK;
}

int agb_selftest_bounded_wait(int poll_limit, int* polls_done, agb_stream_t stream) {
    if (poll_limit < 1 || poll_limit > 100000) return fail(AGB_ERR_INVALID_ARG, "poll_limit %d outside [1, 100000]", poll_limit);
    agb::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(poll_limit, polls_done);
    return after_launch("bounded_wait_selftest");
}

int agb_set_option(const char* key, int64_t value) {
    if (!key) return fail(AGB_ERR_INVALID_ARG, "key is NULL");
    if (!strcmp(key, "stages")) opt_stages = value;
    else if (!strcmp(key, "ctas_per_sm")) opt_ctas_per_sm = value;
    else if (!strcmp(key, "threads")) opt_threads = value;
    else if (!strcmp(key, "force_generic")) opt_force_generic = value;
    else if (!strcmp(key, "ept")) opt_ept = value;
    else if (!strcmp(key, "pdl")) opt_pdl = value;
    else if (!strcmp(key, "softmax_strict")) opt_softmax_strict = value;
    else if (!strcmp(key, "bwd_refill")) opt_bwd_refill = value;  // 1: thread 0 refills after the mid-tile barrier, 2: the last warp out of a slot does
    else if (!strcmp(key, "softmax_two_pass")) opt_softmax_two_pass = value;  // 1: maximum first, then exp; 2: always the one-pass kernel
    else if (!strcmp(key, "free_rows")) opt_free_rows = value;   // 1: the 16-bit forward keeps its block-wide barrier per tile for one-warp rows too
    else if (!strcmp(key, "lone_ring")) opt_lone_ring = value;   // 2: a single CTA per SM may run a two-slot ring
    else if (!strcmp(key, "bf16_strict")) opt_bf16_strict = value;
    else if (!strcmp(key, "bwd_keep")) opt_bwd_keep = value;
    else if (!strcmp(key, "reserve_sms")) opt_reserve_sms = value;
    else if (!strcmp(key, "rows_per_warp")) opt_rpw = value;   // backward, one-warp rows: 0 auto, 1 off, 2..4 forced
    else if (!strcmp(key, "peer_poll_limit"))     // polls before a cross-GPU wait gives up (0 = default, ~2 s)
        opt_peer_poll_limit = value > 0 ? (value < (1 << 22) ? value : (1 << 22)) : (1 << 20);
    else return fail(AGB_ERR_INVALID_ARG, "unknown option '%s'", key);
    return AGB_OK;
}

int agb_describe_launch(int which, int64_t rows, int64_t hidden, int dtype, int fused_add, int64_t out[6]) {
    AGB_TRY(check_common(rows, hidden, dtype));
    if (!out || which < 0 || which > 5) return fail(AGB_ERR_INVALID_ARG, "bad arguments");
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    Plan p;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    if (which <= 2) {
        const int narr = which == kFwd ? (fused_add ? 2 : 1) : (which == kBwd ? (fused_add == 1 ? 3 : 2) : 2);
        bool keep = false;
        if (which == kBwd) plan_bwd(rows, hidden, elem, narr, 1, *d, &p, &keep);
        else plan_launch(static_cast<Which>(which), rows, hidden, elem, narr, 1, *d, &p);
    } else if (which == 3) {   // the same calls as launch_ln_fwd / launch_ln_bwd / launch_ln_jvp
        plan_launch(kFwd, rows, hidden, elem, 1, 0, *d, &p, 0, true);
    } else if (which == 4) {
        plan_launch(kFwd, rows, hidden, elem, fused_add == 1 ? 3 : 2, 0, *d, &p, 0, true);
    } else {
        plan_launch(kJvp, rows, hidden, elem, 2, 0, *d, &p, 0, true);
    }
    if (p.generic) {
        out[0] = generic_grid(rows, *d); out[1] = agb::kGenericThreads; out[2] = 0; out[3] = 0; out[4] = 1; out[5] = 1;
    } else {
        out[0] = p.grid; out[1] = p.block; out[2] = p.smem; out[3] = p.g.stages; out[4] = p.g.rows_per_tile; out[5] = 0;
    }
    return AGB_OK;
}

int agb_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int64_t rows, int64_t hidden, float eps,
                    int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(y, "y", elem));
    AGB_TRY(check_ptr(rstd, "rstd", 4));
    AGB_TRY(check_ptr(gamma, "gamma", elem, false));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_fwd<float>(x, nullptr, gamma, nullptr, y, rstd, rows, hidden, eps, false, st)
                            : launch_fwd<bf16>(x, nullptr, gamma, nullptr, y, rstd, rows, hidden, eps, false, st);
}

int agb_add_rmsnorm_fwd(const void* x, const void* r, const void* gamma, void* h, void* y, float* rstd, int64_t rows,
                        int64_t hidden, float eps, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(r, "r", elem));
    AGB_TRY(check_ptr(h, "h", elem));
    AGB_TRY(check_ptr(y, "y", elem));
    AGB_TRY(check_ptr(rstd, "rstd", 4));
    AGB_TRY(check_ptr(gamma, "gamma", elem, false));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_fwd<float>(x, r, gamma, h, y, rstd, rows, hidden, eps, true, st)
                            : launch_fwd<bf16>(x, r, gamma, h, y, rstd, rows, hidden, eps, true, st);
}

size_t agb_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t hidden, int dtype) {
    (void)rows;
    (void)dtype;
    const DevInfo* d;
    if (hidden <= 0 || device_info(&d) != AGB_OK) return 0;
    return static_cast<size_t>(kMaxCtasPerSm) * d->sms * hidden * sizeof(double);
}

int agb_rmsnorm_bwd(const void* x, const void* gamma, const float* rstd, const void* gy, const void* dx_add, void* dx,
                    void* dgamma, int dgamma_dtype, int accumulate_dgamma, void* workspace, size_t workspace_bytes,
                    int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    const int elem = dtype == AGB_F32 ? 4 : 2;
    if (dgamma && dgamma_dtype != AGB_F32 && dgamma_dtype != AGB_F64)
        return fail(AGB_ERR_INVALID_ARG, "dgamma_dtype must be AGB_F32 or AGB_F64");
    if (dgamma && !gamma) return fail(AGB_ERR_INVALID_ARG, "dgamma requested without gamma");
    if (rows > 0) {
        AGB_TRY(check_ptr(x, "x", elem));
        AGB_TRY(check_ptr(gy, "gy", elem));
        AGB_TRY(check_ptr(dx, "dx", elem));
        AGB_TRY(check_ptr(rstd, "rstd", 4));
        AGB_TRY(check_ptr(dx_add, "dx_add", elem, false));
    }
    AGB_TRY(check_ptr(gamma, "gamma", elem, false));
    AGB_TRY(check_ptr(dgamma, "dgamma", dgamma_dtype == AGB_F64 ? 8 : 4, false));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32
               ? launch_bwd<float>(x, gamma, rstd, gy, dx_add, dx, dgamma, dgamma_dtype, accumulate_dgamma, workspace,
                                   workspace_bytes, rows, hidden, st)
               : launch_bwd<bf16>(x, gamma, rstd, gy, dx_add, dx, dgamma, dgamma_dtype, accumulate_dgamma, workspace,
                                  workspace_bytes, rows, hidden, st);
}

int agb_rmsnorm_bwd_partials(const void* x, const void* gamma, const float* rstd, const void* gy, const void* dx_add,
                             void* dx, void* workspace, size_t workspace_bytes, int64_t rows, int64_t hidden, int dtype,
                             agb_stream_t stream, int* n_partials) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    const int elem = dtype == AGB_F32 ? 4 : 2;
    if (!gamma || !n_partials) return fail(AGB_ERR_INVALID_ARG, "gamma and n_partials are required");
    if (rows > 0) {
        AGB_TRY(check_ptr(x, "x", elem));
        AGB_TRY(check_ptr(gy, "gy", elem));
        AGB_TRY(check_ptr(dx, "dx", elem));
        AGB_TRY(check_ptr(rstd, "rstd", 4));
        AGB_TRY(check_ptr(dx_add, "dx_add", elem, false));
    }
    AGB_TRY(check_ptr(gamma, "gamma", elem));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_bwd<float>(x, gamma, rstd, gy, dx_add, dx, nullptr, AGB_F32, 0, workspace, workspace_bytes,
                                                rows, hidden, st, n_partials)
                            : launch_bwd<bf16>(x, gamma, rstd, gy, dx_add, dx, nullptr, AGB_F32, 0, workspace, workspace_bytes,
                                               rows, hidden, st, n_partials);
}

int agb_dgamma_reduce(const void* partials, int n_partials, int64_t hidden, void* dgamma, int dgamma_dtype, int accumulate,
                      agb_stream_t stream) {
    AGB_RANGE();
    if (hidden <= 0 || n_partials < 0) return fail(AGB_ERR_INVALID_ARG, "hidden=%lld n_partials=%d", (long long)hidden, n_partials);
    if (dgamma_dtype != AGB_F32 && dgamma_dtype != AGB_F64) return fail(AGB_ERR_INVALID_ARG, "dgamma_dtype must be AGB_F32 or AGB_F64");
    AGB_TRY(check_ptr(dgamma, "dgamma", dgamma_dtype == AGB_F64 ? 8 : 4));
    if (n_partials > 0) AGB_TRY(check_ptr(partials, "partials", 8));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n_partials == 0) {   // an empty sum
        if (!accumulate) AGB_CUDA(cudaMemsetAsync(dgamma, 0, hidden * (dgamma_dtype == AGB_F64 ? 8 : 4), st));
        return AGB_OK;
    }
    return launch_dgamma_reduce(static_cast<const double*>(partials), n_partials, hidden, dgamma, dgamma_dtype, accumulate, st,
                                /*behind_backward=*/false);
}

int agb_rmsnorm_bwd_static(const void* x, const void* gamma, const float* rstd, const void* gy, const void* dx_add,
                           void* dx, float* dgamma, int accumulate_dgamma, int64_t rows, int64_t hidden, int dtype,
                           agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    const int elem = dtype == AGB_F32 ? 4 : 2;
    if (dgamma && !gamma) return fail(AGB_ERR_INVALID_ARG, "dgamma requested without gamma");
    if (rows > 0) {
        AGB_TRY(check_ptr(x, "x", elem));
        AGB_TRY(check_ptr(gy, "gy", elem));
        AGB_TRY(check_ptr(dx, "dx", elem));
        AGB_TRY(check_ptr(rstd, "rstd", 4));
        AGB_TRY(check_ptr(dx_add, "dx_add", elem, false));
    }
    AGB_TRY(check_ptr(gamma, "gamma", elem, false));
    AGB_TRY(check_ptr(dgamma, "dgamma", 4, false));
    void* scratch = nullptr;
    if (gamma && dgamma) {
        const DevInfo* d;
        AGB_TRY(device_info(&d));
        const size_t need = static_cast<size_t>(max_partials(*d)) * hidden * sizeof(double);
        if (need > kStaticScratchBytes)
            return fail(AGB_ERR_WORKSPACE,
                        "hidden=%lld needs %zu bytes of scratch but the built-in array holds %zu "
                        "(largest hidden on this device: %zu); use agb_rmsnorm_bwd with a caller workspace",
                        (long long)hidden, need, kStaticScratchBytes,
                        kStaticScratchBytes / (static_cast<size_t>(max_partials(*d)) * sizeof(double)));
        AGB_TRY(static_scratch_for_current_device(&scratch));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32
               ? launch_bwd<float>(x, gamma, rstd, gy, dx_add, dx, dgamma, AGB_F32, accumulate_dgamma, scratch,
                                   kStaticScratchBytes, rows, hidden, st)
               : launch_bwd<bf16>(x, gamma, rstd, gy, dx_add, dx, dgamma, AGB_F32, accumulate_dgamma, scratch,
                                  kStaticScratchBytes, rows, hidden, st);
}

int agb_dgamma_finalize(const double* sum, float* dgamma, int64_t hidden, int accumulate, agb_stream_t stream) {
    AGB_RANGE();
    if (hidden <= 0) return fail(AGB_ERR_INVALID_ARG, "hidden=%lld", (long long)hidden);
    AGB_TRY(check_ptr(sum, "sum", 8));
    AGB_TRY(check_ptr(dgamma, "dgamma", 4));
    agb::dgamma_finalize_kernel<<<(unsigned)((hidden + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sum, dgamma, (int)hidden, accumulate);
    return after_launch("dgamma_finalize");
}

int agb_rmsnorm_jvp(const void* x, const void* gamma, const float* rstd, const void* tx, const void* tgamma, void* ty,
                    int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(tx, "tx", elem));
    AGB_TRY(check_ptr(ty, "ty", elem));
    AGB_TRY(check_ptr(rstd, "rstd", 4));
    AGB_TRY(check_ptr(gamma, "gamma", elem, false));
    AGB_TRY(check_ptr(tgamma, "tgamma", elem, false));
    if (tgamma && !gamma) return fail(AGB_ERR_INVALID_ARG, "tgamma given without gamma");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_jvp<float>(x, gamma, rstd, tx, tgamma, ty, rows, hidden, st)
                            : launch_jvp<bf16>(x, gamma, rstd, tx, tgamma, ty, rows, hidden, st);
}

namespace {
int softmax_family(int mode, const void* z, const void* t, const void* rowscale, const void* add, void* out, void* out_row,
                   int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(z, "z", elem));
    AGB_TRY(check_ptr(t, "t", elem, mode == 3));
    AGB_TRY(check_ptr(rowscale, "gy", elem, mode == 2));
    AGB_TRY(check_ptr(add, "add", elem, false));
    AGB_TRY(check_ptr(out, "out", elem, mode == 0 || mode == 2));
    AGB_TRY(check_ptr(out_row, "out", elem, mode == 1 || mode == 3));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_softmax_fwd<float>(mode, z, t, rowscale, add, out, out_row, rows, hidden, st)
                            : launch_softmax_fwd<bf16>(mode, z, t, rowscale, add, out, out_row, rows, hidden, st);
}
}  // namespace

int agb_layernorm_jvp(const void* y, const void* t, const float* var, void* ty, int64_t rows, int64_t hidden, float eps,
                      int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(y, "y", elem));
    AGB_TRY(check_ptr(t, "t", elem));
    AGB_TRY(check_ptr(ty, "ty", elem));
    AGB_TRY(check_ptr(var, "var", 4));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_ln_jvp<float>(y, t, var, ty, rows, hidden, eps, st)
                            : launch_ln_jvp<bf16>(y, t, var, ty, rows, hidden, eps, st);
}

int agb_softmax_row_fwd(const void* z, void* y, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    return softmax_family(0, z, nullptr, nullptr, nullptr, y, nullptr, rows, hidden, dtype, stream);
}
int agb_logsumexp_row_fwd(const void* z, void* out, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    return softmax_family(1, z, nullptr, nullptr, nullptr, nullptr, out, rows, hidden, dtype, stream);
}
int agb_logsumexp_row_bwd(const void* z, const void* gy, const void* dz_add, void* dz, int64_t rows, int64_t hidden,
                          int dtype, agb_stream_t stream) {
    return softmax_family(2, z, nullptr, gy, dz_add, dz, nullptr, rows, hidden, dtype, stream);
}
int agb_logsumexp_row_jvp(const void* z, const void* tz, void* out, int64_t rows, int64_t hidden, int dtype,
                          agb_stream_t stream) {
    return softmax_family(3, z, tz, nullptr, nullptr, nullptr, out, rows, hidden, dtype, stream);
}
int agb_softmax_row_bwd(const void* y, const void* g, const void* dz_add, void* dz, int64_t rows, int64_t hidden,
                        int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(y, "y", elem));
    AGB_TRY(check_ptr(g, "g", elem));
    AGB_TRY(check_ptr(dz, "dz", elem));
    AGB_TRY(check_ptr(dz_add, "dz_add", elem, false));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_softmax_bwd<float>(y, g, dz_add, dz, rows, hidden, st)
                            : launch_softmax_bwd<bf16>(y, g, dz_add, dz, rows, hidden, st);
}

int agb_residual_add(const void* a, const void* b, void* out, int64_t n, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    if (n < 0) return fail(AGB_ERR_INVALID_ARG, "n=%lld", (long long)n);
    if (dtype != AGB_F32 && dtype != AGB_BF16) return fail(AGB_ERR_UNSUPPORTED, "dtype %d", dtype);
    if (n == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(a, "a", elem));
    AGB_TRY(check_ptr(b, "b", elem));
    AGB_TRY(check_ptr(out, "out", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    const int vec = aligned16(a) && aligned16(b) && aligned16(out);
    const int grid = ew_grid(n / (16 / elem) + 1, *d);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == AGB_F32) agb::residual_add_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (float*)out, n, vec);
    else agb::residual_add_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n, vec);
    return after_launch("residual_add");
}

int agb_vjp_add(void* ga, void* gb, const void* gy, int64_t n, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    if (n < 0) return fail(AGB_ERR_INVALID_ARG, "n=%lld", (long long)n);
    if (dtype != AGB_F32 && dtype != AGB_BF16) return fail(AGB_ERR_UNSUPPORTED, "dtype %d", dtype);
    if (n == 0 || (!ga && !gb)) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(gy, "gy", elem));
    AGB_TRY(check_ptr(ga, "ga", elem, false));
    AGB_TRY(check_ptr(gb, "gb", elem, false));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    const int vec = aligned16(gy) && (!ga || aligned16(ga)) && (!gb || aligned16(gb));
    const int grid = ew_grid(n / (16 / elem) + 1, *d);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == AGB_F32) agb::vjp_add_kernel<float><<<grid, 256, 0, st>>>((float*)ga, (float*)gb, (const float*)gy, n, vec);
    else agb::vjp_add_kernel<bf16><<<grid, 256, 0, st>>>((bf16*)ga, (bf16*)gb, (const bf16*)gy, n, vec);
    return after_launch("vjp_add");
}

int agb_scale_lastdim(const void* a, const void* g, void* out, int64_t rows, int64_t hidden, int dtype,
                      agb_stream_t stream) {
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(a, "a", elem));
    AGB_TRY(check_ptr(g, "g", elem));
    AGB_TRY(check_ptr(out, "out", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    const int vec = aligned16(a) && aligned16(g) && aligned16(out) && (hidden * elem) % 16 == 0;
    const int grid = ew_grid(rows * hidden / (16 / elem) + 1, *d);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == AGB_F32) agb::scale_lastdim_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)g, (float*)out, rows, (int)hidden, vec);
    else agb::scale_lastdim_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)a, (const bf16*)g, (bf16*)out, rows, (int)hidden, vec);
    return after_launch("scale_lastdim");
}

int agb_binary_broadcast(int op, const void* a, const void* b, void* out, int64_t rows, int64_t hidden, int b_mode,
                         int dtype, agb_stream_t stream) {
    AGB_TRY(check_common(rows, hidden, dtype));
    if (op < 0 || op > 1 || b_mode < 0 || b_mode > 3) return fail(AGB_ERR_INVALID_ARG, "op %d b_mode %d", op, b_mode);
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(a, "a", elem));
    AGB_TRY(check_ptr(b, "b", elem));
    AGB_TRY(check_ptr(out, "out", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = ew_grid(rows * hidden, *d);
    if (dtype == AGB_F32) agb::binary_broadcast_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (float*)out, rows, (int)hidden, b_mode, op);
    else agb::binary_broadcast_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)a, (const bf16*)b, (bf16*)out, rows, (int)hidden, b_mode, op);
    return after_launch("binary_broadcast");
}

int agb_accumulate_broadcast(void* dst, const void* src, int64_t rows, int64_t hidden, int src_mode, float scale,
                             int dtype, agb_stream_t stream) {
    AGB_TRY(check_common(rows, hidden, dtype));
    if (src_mode < 0 || src_mode > 3) return fail(AGB_ERR_INVALID_ARG, "src_mode %d", src_mode);
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(dst, "dst", elem));
    AGB_TRY(check_ptr(src, "src", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = ew_grid(rows * hidden, *d);
    const int use_scale = scale != 1.0f;
    if (dtype == AGB_F32) agb::accumulate_broadcast_kernel<float><<<grid, 256, 0, st>>>((float*)dst, (const float*)src, rows, (int)hidden, src_mode, scale, use_scale);
    else agb::accumulate_broadcast_kernel<bf16><<<grid, 256, 0, st>>>((bf16*)dst, (const bf16*)src, rows, (int)hidden, src_mode, scale, use_scale);
    return after_launch("accumulate_broadcast");
}

size_t agb_mul_reduce_workspace_bytes(int64_t rows, int64_t hidden) {
    (void)rows;
    const DevInfo* d;
    if (hidden <= 0 || device_info(&d) != AGB_OK) return 0;
    const size_t col = static_cast<size_t>(max_partials(*d)) * hidden * sizeof(double);
    return col > 1024 * sizeof(double) ? col : 1024 * sizeof(double);
}

}  // extern "C"

template <typename T>
static int launch_mul_reduce(const void* g, const void* a, void* out, int64_t rows, int64_t hidden, int out_mode,
                             int accumulate, double* ws, cudaStream_t st) {
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    if (out_mode == AGB_BCAST_LASTVEC) {
        int P = static_cast<int>(rows < max_partials(*d) ? rows : max_partials(*d));
        const int64_t rpc = (rows + P - 1) / P;
        P = static_cast<int>((rows + rpc - 1) / rpc);
        dim3 grid((unsigned)((hidden + 255) / 256), (unsigned)P);
        agb::mul_colsum_partial_kernel<T><<<grid, 256, 0, st>>>((const T*)g, (const T*)a, ws, rows, (int)hidden, rpc);
        AGB_TRY(after_launch("mul_colsum_partial"));
        agb::colsum_finish_kernel<T><<<(unsigned)((hidden + 255) / 256), 256, 0, st>>>(ws, P, (int)hidden, (T*)out, accumulate);
        return after_launch("colsum_finish");
    }
    if (out_mode == AGB_BCAST_ROWSTAT) {
        agb::mul_rowsum_kernel<T><<<generic_grid(rows, *d), 256, 0, st>>>((const T*)g, (const T*)a, (T*)out, rows, (int)hidden, accumulate);
        return after_launch("mul_rowsum");
    }
    int nb;
    int64_t chunk;
    const int64_t n = rows * hidden;
    int64_t nbl = (n + 16383) / 16384;
    if (nbl > 1024) nbl = 1024;
    if (nbl < 1) nbl = 1;
    chunk = (n + nbl - 1) / nbl;
    nb = static_cast<int>((n + chunk - 1) / chunk);
    agb::mul_sumall_stage1<T><<<nb, 256, 0, st>>>((const T*)g, (const T*)a, ws, n, chunk);
    AGB_TRY(after_launch("mul_sumall_stage1"));
    agb::sumall_finish_kernel<T><<<1, 32, 0, st>>>(ws, nb, (T*)out, accumulate);
    return after_launch("sumall_finish");
}

extern "C" {

int agb_mul_reduce(const void* g, const void* a, void* out, int64_t rows, int64_t hidden, int out_mode, int accumulate,
                   void* workspace, size_t workspace_bytes, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (out_mode < AGB_BCAST_LASTVEC || out_mode > AGB_BCAST_SCALAR) return fail(AGB_ERR_INVALID_ARG, "out_mode %d", out_mode);
    if (rows == 0) return fail(AGB_ERR_INVALID_ARG, "rows == 0");
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(g, "g", elem));
    AGB_TRY(check_ptr(a, "a", elem, false));
    AGB_TRY(check_ptr(out, "out", elem));
    if (out_mode != AGB_BCAST_ROWSTAT) {
        if (!workspace || workspace_bytes < agb_mul_reduce_workspace_bytes(rows, hidden))
            return fail(AGB_ERR_WORKSPACE, "workspace %zu bytes, need %zu", workspace_bytes, agb_mul_reduce_workspace_bytes(rows, hidden));
        AGB_TRY(check_ptr(workspace, "workspace", 8));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_mul_reduce<float>(g, a, out, rows, hidden, out_mode, accumulate, (double*)workspace, st)
                            : launch_mul_reduce<bf16>(g, a, out, rows, hidden, out_mode, accumulate, (double*)workspace, st);
}

int agb_layernorm_fwd(const void* x, void* y, float* mean, float* var, int64_t rows, int64_t hidden, float eps,
                      int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(y, "y", elem));
    AGB_TRY(check_ptr(mean, "mean", 4));
    AGB_TRY(check_ptr(var, "var", 4));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_ln_fwd<float>(x, y, mean, var, rows, hidden, eps, st)
                            : launch_ln_fwd<bf16>(x, y, mean, var, rows, hidden, eps, st);
}

int agb_layernorm_bwd(const void* x, const float* mean, const float* var, const void* gy, const void* dx_add, void* dx,
                      int64_t rows, int64_t hidden, float eps, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(gy, "gy", elem));
    AGB_TRY(check_ptr(dx, "dx", elem));
    AGB_TRY(check_ptr(mean, "mean", 4));
    AGB_TRY(check_ptr(var, "var", 4));
    AGB_TRY(check_ptr(dx_add, "dx_add", elem, false));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == AGB_F32 ? launch_ln_bwd<float>(x, mean, var, gy, dx_add, dx, rows, hidden, eps, st)
                            : launch_ln_bwd<bf16>(x, mean, var, gy, dx_add, dx, rows, hidden, eps, st);
}

int agb_sgd_step(void* param, const void* grad, int64_t n, float learning_rate, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    if (n < 0) return fail(AGB_ERR_INVALID_ARG, "n=%lld", (long long)n);
    if (dtype != AGB_F32 && dtype != AGB_BF16) return fail(AGB_ERR_UNSUPPORTED, "dtype %d", dtype);
    if (n == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(param, "param", elem));
    AGB_TRY(check_ptr(grad, "grad", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == AGB_F32) agb::sgd_step_kernel<float><<<ew_grid(n, *d), 256, 0, st>>>((float*)param, (const float*)grad, n, -learning_rate);
    else agb::sgd_step_kernel<bf16><<<ew_grid(n, *d), 256, 0, st>>>((bf16*)param, (const bf16*)grad, n, -learning_rate);
    return after_launch("sgd_step");
}

int agb_adam_step(float* param, const float* grad, float* m, float* v, int64_t n, float beta1, float beta2,
                  float alpha_eff, float eps_eff, agb_stream_t stream) {
    AGB_RANGE();
    if (n < 0) return fail(AGB_ERR_INVALID_ARG, "n=%lld", (long long)n);
    if (n == 0) return AGB_OK;
    AGB_TRY(check_ptr(param, "param", 4));
    AGB_TRY(check_ptr(grad, "grad", 4));
    AGB_TRY(check_ptr(m, "m", 4));
    AGB_TRY(check_ptr(v, "v", 4));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    agb::adam_step_kernel<<<ew_grid(n, *d), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        param, grad, m, v, n, beta1, beta2, 1.0f - beta1, 1.0f - beta2, alpha_eff, eps_eff);
    return after_launch("adam_step");
}

int agb_row_reduce(int op, const void* x, void* out, int64_t rows, int64_t hidden, int dtype, agb_stream_t stream) {
    AGB_RANGE();
    AGB_TRY(check_common(rows, hidden, dtype));
    if (op < AGB_REDUCE_SUM || op > AGB_REDUCE_MAX) return fail(AGB_ERR_INVALID_ARG, "op %d", op);
    if (rows == 0) return AGB_OK;
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(out, "out", elem));
    const DevInfo* d;
    AGB_TRY(device_info(&d));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool wide = hidden >= 1024;
    const int rpc = wide ? 1 : 8;
    int64_t g = (rows + rpc - 1) / rpc;
    const int64_t cap = static_cast<int64_t>(d->sms) * 8;
    const int grid = static_cast<int>(g < cap ? g : cap);
    // rows of whole 16-byte vectors at an aligned base: the vector-load kernels
    if (aligned16(x) && (hidden * elem) % 16 == 0 && !opt_force_generic.load()) {
#define AGB_ROW_REDUCE_VEC(T, TPR)                                                                                       \
    do {                                                                                                                 \
        if (op == AGB_REDUCE_MAX) agb::row_reduce_vec_kernel<T, TPR, true><<<grid, 256, 0, st>>>((const T*)x, (T*)out, rows, (int)hidden, op); \
        else agb::row_reduce_vec_kernel<T, TPR, false><<<grid, 256, 0, st>>>((const T*)x, (T*)out, rows, (int)hidden, op); \
    } while (0)
        if (dtype == AGB_F32) {
            if (wide) AGB_ROW_REDUCE_VEC(float, 256);
            else AGB_ROW_REDUCE_VEC(float, 32);
        } else {
            if (wide) AGB_ROW_REDUCE_VEC(bf16, 256);
            else AGB_ROW_REDUCE_VEC(bf16, 32);
        }
#undef AGB_ROW_REDUCE_VEC
        return after_launch("row_reduce_vec");
    }
    if (dtype == AGB_F32) {
        if (wide) agb::row_reduce_kernel<float, 256><<<grid, 256, 0, st>>>((const float*)x, (float*)out, rows, (int)hidden, op);
        else agb::row_reduce_kernel<float, 32><<<grid, 256, 0, st>>>((const float*)x, (float*)out, rows, (int)hidden, op);
    } else {
        if (wide) agb::row_reduce_kernel<bf16, 256><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)out, rows, (int)hidden, op);
        else agb::row_reduce_kernel<bf16, 32><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)out, rows, (int)hidden, op);
    }
    return after_launch("row_reduce");
}

static inline void reduce_all_shape(int64_t n, int* nblocks, int64_t* chunk) {
    // a function of n only, so the summation order (and the result) depends on nothing else
    int64_t nb = (n + 16383) / 16384;
    if (nb > 1024) nb = 1024;
    if (nb < 1) nb = 1;
    *chunk = ((n + nb - 1) / nb + 7) / 8 * 8;   // whole 16-byte vectors per block, for either element size
    *nblocks = static_cast<int>((n + *chunk - 1) / *chunk);
    if (*nblocks < 1) *nblocks = 1;
}

size_t agb_reduce_all_workspace_bytes(int64_t n) {
    (void)n;
    return 1024 * sizeof(double);
}

int agb_reduce_all(int op, const void* x, void* out, int64_t n, int dtype, void* workspace, size_t workspace_bytes,
                   agb_stream_t stream) {
    AGB_RANGE();
    if (n <= 0) return fail(AGB_ERR_INVALID_ARG, "n=%lld", (long long)n);
    if (dtype != AGB_F32 && dtype != AGB_BF16) return fail(AGB_ERR_UNSUPPORTED, "dtype %d", dtype);
    if (op != AGB_REDUCE_SUM && op != AGB_REDUCE_MEAN) return fail(AGB_ERR_INVALID_ARG, "op %d (sum or mean)", op);
    const int elem = dtype == AGB_F32 ? 4 : 2;
    AGB_TRY(check_ptr(x, "x", elem));
    AGB_TRY(check_ptr(out, "out", elem));
    if (!workspace || workspace_bytes < agb_reduce_all_workspace_bytes(n))
        return fail(AGB_ERR_WORKSPACE, "workspace %zu bytes, need %zu", workspace_bytes, agb_reduce_all_workspace_bytes(n));
    AGB_TRY(check_ptr(workspace, "workspace", 8));
    int nb;
    int64_t chunk;
    reduce_all_shape(n, &nb, &chunk);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    double* part = static_cast<double*>(workspace);
    if (dtype == AGB_F32) {
        agb::reduce_all_stage1<float><<<nb, 256, 0, st>>>((const float*)x, part, n, chunk);
        AGB_TRY(after_launch("reduce_all_stage1"));
        agb::reduce_all_stage2<float><<<1, 32, 0, st>>>(part, nb, (float*)out, n, op);
    } else {
        agb::reduce_all_stage1<bf16><<<nb, 256, 0, st>>>((const bf16*)x, part, n, chunk);
        AGB_TRY(after_launch("reduce_all_stage1"));
        agb::reduce_all_stage2<bf16><<<1, 32, 0, st>>>(part, nb, (bf16*)out, n, op);
    }
    return after_launch("reduce_all_stage2");
}

}  // extern "C"
#include "agb_shard.cuh"
#include "agb_peer.cuh"
#include "agb_host.cuh"
