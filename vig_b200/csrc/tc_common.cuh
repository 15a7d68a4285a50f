// Device-side PTX wrappers (mbarrier, TMA, tcgen05, TMEM) and host-side tensor-map helpers shared by the
// tensor-core bi-GLA kernels.
#pragma once
#include <cuda.h>
#include <mutex>
#include <type_traits>
#include "common.cuh"

namespace vig {
namespace tc {

constexpr int CHUNK = 128;            // tokens per chunk = rows of one MMA tile
constexpr float MAX_EXPONENT = 80.f;  // exp() arguments of the factorisation are clamped to +-80

struct TcMaps { CUtensorMap q, k, v, gf, gb; };

// ---------------------------------------------------------------------------------------------------
// PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a hardware-defined time when the phase is pending;
// this form answers at once): for polls issued ahead of time, whose answer is looked at later.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// The same test, but the hardware may park the thread for up to `ns` nanoseconds while the phase is pending and
// wakes it when the phase completes: a waiting warp then issues almost no instructions.
__device__ __forceinline__ uint32_t mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// ask for a tile to be brought into L2 ahead of the load that will need it
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// tiled stores from shared memory: plain, and with an element-wise add at the destination (done in L2)
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t src) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// untiled bulk copies: a 16 KB operand tile to / from its parking slot in global memory
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t ssrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(ssrc), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void mbar_arrive_plain(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Low word: start address (bits 0-13, in 16-byte units) and leading byte offset 1 (bits 16-29; unused for one
// 128-byte atom column).  High word: stride byte offset 1024 >> 4 (bits 32-45), descriptor version 1 (bit 46),
// SWIZZLE_128B (bits 61-63).
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t make_desc(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
// a_lo / b_lo: low words of the shared-memory descriptors (see make_desc_lo); the high word is the same constant
// for every tile of this kernel, so an MMA costs one integer add per operand to set up.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(DESC_HI) : "memory");
}
// The same MMA with the A operand read from tensor memory: lane i of [a_tmem] holds row i of A, one 32-bit column holds two
// consecutive K elements (the lower-indexed one in the low half), so a K = 16 step consumes 8 columns.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "mov.b64 db, {%2, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(DESC_HI) : "memory");
}
// registers -> tensor memory, 32 lanes x 16 consecutive 32-bit columns: thread i of the warp writes lane (base lane + i)
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart (both for K-major
// tiles with 128-byte rows along K and for MN-major tiles with 128-byte rows along M/N).
// Instruction descriptor: fp32 accumulate, A/B format (0 fp16, 1 bf16), major-ness (0 K, 1 MN), N, M.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t a_mn, uint32_t b_mn, uint32_t M, uint32_t N) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Byte offset of bf16 element (row, col) in a K-major / MN-major tile with 128-byte rows and 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t col_bytes) {
    return row * 128 + ((((col_bytes >> 4) ^ (row & 7)) << 4) | (col_bytes & 15));
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    static constexpr uint32_t FMT = 1;
    __device__ static uint32_t pack(float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); }
    __device__ static float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
};
template <> struct Pack2<__half> {
    static constexpr uint32_t FMT = 0;
    __device__ static uint32_t pack(float a, float b) { __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); }
    __device__ static float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
};

struct Waiter {
    volatile int* abort_flag;
    int32_t* status;
    // Bounded wait: about a second at most, then flag the CTA as aborted so that no later wait spins.  The polling
    // loop must stay rolled (a kernel has dozens of wait sites and the instruction cache is a bottleneck of these
    // kernels) and parks the thread in hardware between polls (spinning warps would take issue slots from the others).
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity) const {
        if (mbar_try_wait(bar, parity)) return;
#pragma unroll 1
        for (uint32_t i = 0; i < (1u << 19); ++i) {
            if (mbar_try_wait_parked(bar, parity, 2000u)) return;
            if (*abort_flag) return;
        }
        *abort_flag = 1;
        if (status) atomicOr(status, 1);
    }
    // The same bounded wait in as few instructions as it takes, for kernels with dozens of wait sites that are bound by
    // the instruction cache: a run-out only raises the CTA's abort flag; the kernel ORs the status word once, at its end.
    __device__ __forceinline__ void wait_lite(uint32_t bar, uint32_t parity) const {
#pragma unroll 1
        for (uint32_t i = 0; !mbar_try_wait_parked(bar, parity, 2000u); ++i)
            if (i >= (1u << 19) || *abort_flag) { *abort_flag = 1; break; }
    }
};

// A pair of fp32 values in one 64-bit register and the two-wide fp32 arithmetic of sm_100 on it (add / mul / fma .f32x2:
// one instruction for two values, each lane the IEEE operation, so results equal the scalar form's).  For loops that are
// bound by instruction issue.
typedef unsigned long long F2;
__device__ __forceinline__ F2 f2_make(float lo, float hi) { F2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ float f2_lo(F2 v) { float lo, hi; asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); return lo; }
__device__ __forceinline__ float f2_hi(F2 v) { float lo, hi; asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); return hi; }
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) { F2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) { F2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) { F2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

// single-instruction exp2 / log2 (flush-to-zero forms: no denormal fix-up code around the MUFU)
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
constexpr float MAX_EXPONENT2 = MAX_EXPONENT * LOG2E;   // the exponent bound in log2 units

// Log-gate in LOG2 units.  From a raw logit: logsigmoid(x) = min(x,0) - log(1 + exp(-|x|)), here with y = x log2(e):
// min(y,0) - log2(1 + 2^-|y|), times 1/normalizer.  From a log-gate: x log2(e).
__device__ __forceinline__ float fast_gate2(float x, bool raw_logits, float inv_norm) {
    const float y = x * LOG2E;
    return raw_logits ? (fminf(y, 0.f) - lg2(1.f + ex2(-fabsf(y)))) * inv_norm : y;
}

// Log-gate in log2 units, branch-free and short: from a raw logit x, logsigmoid(x) / norm = -log2(1 + 2^(-x log2 e)) / norm
// (for very negative x the power overflows to +inf and the gate to -inf, which the exponent clamp catches and flags
// like any other gate beyond the factorisation range); from a log-gate, x log2 e.
__device__ __forceinline__ float gate2_short(float x, bool raw_logits, float neg_inv_norm) {
    const float y = x * LOG2E;
    const float sp = lg2(1.f + ex2(-y)) * neg_inv_norm;
    return raw_logits ? sp : y;
}

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}


// ---------------------------------------------------------------------------------------------------
// Host side: tensor maps through the driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Tensor maps are cached: a model calls the same kernels with the same buffers and shapes layer after layer and step
// after step, and encoding five maps per scan launch is host time that shows at small problem sizes.  Key = every
// argument of the encoding (base pointer, dims, strides, box, type, swizzle); direct-mapped table behind a mutex.
struct MapKey {
    const void* base;
    uint64_t dims[4], strides[3];
    uint32_t box[4];
    int rank, dtype, swizzle;
    bool operator==(const MapKey& o) const {
        if (base != o.base || rank != o.rank || dtype != o.dtype || swizzle != o.swizzle) return false;
        for (int i = 0; i < 4; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        for (int i = 0; i < 3; ++i) if (strides[i] != o.strides[i]) return false;
        return true;
    }
    uint64_t hash() const {
        uint64_t h = 1469598103934665603ull;
        auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; h ^= h >> 29; };
        mix(reinterpret_cast<uint64_t>(base));
        for (int i = 0; i < 4; ++i) { mix(dims[i]); mix(box[i]); }
        for (int i = 0; i < 3; ++i) mix(strides[i]);
        mix((uint64_t)rank * 64 + (uint64_t)dtype * 8 + (uint64_t)swizzle);
        return h;
    }
};

inline bool encode_cached(CUtensorMap* m, const MapKey& key) {
    constexpr int SLOTS = 1024;
    struct Slot { bool used; MapKey key; CUtensorMap map; };
    static Slot* table = new Slot[SLOTS]();
    static std::mutex mu;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const int slot = (int)(key.hash() % SLOTS);
    std::lock_guard<std::mutex> lock(mu);
    Slot& s = table[slot];
    if (s.used && s.key == key) { *m = s.map; return true; }
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
    for (int i = 0; i < 4; ++i) { dims[i] = key.dims[i]; box[i] = key.box[i]; }
    for (int i = 0; i < 3; ++i) strides[i] = key.strides[i];
    CUresult r = fn(m, key.dtype == VIG_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)key.rank,
                    const_cast<void*>(key.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    key.swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    s.used = true; s.key = key; s.map = *m;
    return true;
}

// [B,H,L,d] view with element strides s = (b, h, l): box of 128 tokens x d channels of one (b, h).
// ``box_d`` > d: the box is wider than the tensor's channel extent and the channels past d arrive as zeros (TMA fill).
inline bool make_map(CUtensorMap* m, const void* base, const int64_t* s, int B, int H, int L, int d, int dtype, bool swizzle128, int box_d = 0) {
    MapKey key{};
    key.base = base; key.rank = 4; key.dtype = dtype; key.swizzle = swizzle128 ? 1 : 0;
    key.dims[0] = (uint64_t)d; key.dims[1] = (uint64_t)L; key.dims[2] = (uint64_t)H; key.dims[3] = (uint64_t)B;
    key.strides[0] = (uint64_t)s[2] * 2; key.strides[1] = (uint64_t)s[1] * 2; key.strides[2] = (uint64_t)s[0] * 2;
    key.box[0] = (uint32_t)(box_d > 0 ? box_d : d); key.box[1] = CHUNK; key.box[2] = 1; key.box[3] = 1;
    return encode_cached(m, key);
}

// Row-major [rows, cols] matrix with leading dimension ld (elements): boxes of box_rows x 64 columns, 128-byte swizzle.
inline bool make_map_2d(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int dtype) {
    MapKey key{};
    key.base = base; key.rank = 2; key.dtype = dtype; key.swizzle = 1;
    key.dims[0] = (uint64_t)cols; key.dims[1] = (uint64_t)rows;
    key.strides[0] = (uint64_t)ld * 2;
    key.box[0] = 64; key.box[1] = (uint32_t)box_rows;
    return encode_cached(m, key);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of on every launch.
inline cudaError_t ensure_smem_attr(const void* kern, int bytes) {
    struct Entry { const void* kern; int dev; int bytes; };
    static std::mutex mu;
    static Entry entries[256];
    static int count = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    Entry* hit = nullptr;
    for (int i = 0; i < count; ++i)
        if (entries[i].kern == kern && entries[i].dev == dev) { hit = &entries[i]; break; }
    if (hit && hit->bytes >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    if (hit) hit->bytes = bytes;
    else if (count < 256) entries[count++] = Entry{kern, dev, bytes};
    return cudaSuccess;
}

inline bool tma_ok(const void* base, const int64_t* s, int B, int H) {
    if (!base) return true;
    if (reinterpret_cast<uintptr_t>(base) & 15) return false;
    for (int i = 0; i < 3; ++i) {
        const bool unused = (i == 0 && B == 1) || (i == 1 && H == 1);
        if (s[i] <= 0 && !unused) return false;
        if ((s[i] * 2) % 16) return false;
    }
    return true;
}


}  // namespace tc
}  // namespace vig
