// Bi-directional gated linear attention, warp-specialised "wavefront" form for large batches (tcgen05 + TMEM).
//
// Work item = (sequence b*h, run of 2, 4 or 8 chunks of 128 tokens, direction).  Items are drawn from a ticket counter
// in wavefront order: step w holds the w-th item of every chain (a forward chain counts its chunks from the start of the
// sequence, a backward chain from its end, both through the same schedule of item lengths, shorter at the end), so the
// state that enters an item was produced by an item with a smaller ticket, which is running or done.  States pass from
// item to item through a two-slot mailbox per (sequence, direction) in global memory; the two directions of a chunk
// meet in the output tensor: the direction that is scheduled first stores its half, the other adds to it with a TMA
// reduction once the first has raised the chunk's flag.
//
// One persistent CTA per SM runs a pipeline over its stream of chunk iterations, roles decoupled by mbarriers:
//
//   load thread       work tickets; TMA loads of q, k, gates, v into a 3-stage ring
//   MMA warp          all tcgen05.mma issue (the whole warp walks the loops, lane 0 issues)
//   16 worker warps   one instruction stream per trip: for iteration m the gate transform and cumulative log-gates (in
//                     registers; group sums exchanged through shared memory, every warp forms its own offset from them),
//                     then q * 2^(G_i - G_ref) and k * 2^(G_ref - G_j) IN PLACE over the raw tiles; in between, the scores
//                     of iteration m-1 from tensor memory, masked, back to tensor memory as packed 16-bit pairs, and the
//                     output accumulator of iteration m-2 from tensor memory to a 16-bit staging tile in shared memory
//   store thread      staging tile -> global by TMA (store, or reduction onto the other direction's half); chunk flags
//   4 state warps     S <- 2^G_last S + 2^(G_last - G_ref) K~^T V in registers; bf16 state operand; mailbox
//
// Per iteration m (one chunk of 128 tokens, one direction), on the tensor core:
//   P  = Q~ K~^T                (128x128x64)   then masked by the worker warps
//   U  = K~^T V                 ( 64x 64x128)  right behind it: the state chain waits for nothing else
//   O  = Q~ (2^G_ref S_in)      (128x 64x64)   skipped when S_in is exactly zero
//   O += P V                    (128x 64x128)  P read from tensor memory
// Only the state chain (U -> S -> state operand -> next chunk's second product) is sequential; everything else of
// the following iterations runs ahead as far as the rings allow.
// A call without an output (end states and summed log-gates only) runs the SO instantiation: no q, no P, no O, no masking,
// no staging.
//
// Every wait (mbarrier, mailbox counter, chunk flag) is bounded; when one runs out the CTA sets bit 0 of the status
// word, stops waiting on anything else, drains its control flow and frees its tensor memory.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int WDK = 64, WDV = 64;
// A work item is a run of 2, 4 or 8 chunks of one (sequence, direction) chain: a longer run has fewer hand-overs (state
// mailbox, ring restart: 0.361 -> 0.340 -> 0.337 ms at 64 x 3 sequences of 4096 tokens for 2 -> 4 -> 8 chunks), a shorter one
// gives the wavefront more items to balance over the SMs.  The host picks the length per call (wave_seg_chunks).
constexpr int W_SEG_CHUNKS_MIN = 2, W_SEG_CHUNKS_MAX = 8;
// six warpgroups: workers x4, state, control (MMA warp, load thread, store thread)
constexpr int W_PREP_WARPS = 16, W_STATE_WARP0 = 16, W_CTRL_WARP0 = 20, W_THREADS = 24 * 32;
constexpr int W_MMA_WARP = W_CTRL_WARP0, W_LOAD_WARP = W_CTRL_WARP0 + 1, W_STORE_WARP = W_CTRL_WARP0 + 2;
constexpr int W_STAGES = 3;
// Registers per thread.  The kernel is compiled and launched with W_REGS_BASE for all six warpgroups; the control
// warpgroup gives most of its share back and the state warpgroup takes it.  An increase waits until the registers are
// there, so the shares must never add up to more than was launched with.
constexpr int W_REGS_BASE = 80, W_REGS_WORK = W_REGS_BASE, W_REGS_STATE = 96, W_REGS_CTRL = 40;
static_assert(4 * W_REGS_WORK + W_REGS_STATE + W_REGS_CTRL <= 6 * W_REGS_BASE, "register shares exceed the launch allocation");
constexpr int W_TILE = CHUNK * 128;                           // 16 KB: 128 rows x 128 B
constexpr int W_STAGE_B = 4 * W_TILE;                         // q | k | gates | v
constexpr int WS_Q = 0, WS_K = W_TILE, WS_G = 2 * W_TILE, WS_V = 3 * W_TILE;
constexpr int WO_X = W_STAGES * W_STAGE_B;                    // score tile of key columns 64..127 (0..63 go over the dead gate tile)
constexpr int WO_ST = WO_X + W_TILE;                          // bf16 state operand, 64 rows x 128 B
constexpr int WO_PART = WO_ST + 64 * 128;                     // fp32 [2][16][64]: group sums of log-gates, turned in place into group offsets
constexpr int WO_VEC = WO_PART + 2 * W_PREP_WARPS * 64 * 4;   // fp32 [4][2][64]: G_ref, G_last per iteration
constexpr int WO_ITEMS = WO_VEC + 4 * 2 * 64 * 4;             // ring of 8 work items x 8 ints
constexpr int WO_BAR = WO_ITEMS + 8 * 32;
constexpr int WO_MISC = WO_BAR + 32 * 8;                      // tmem base, abort flag
constexpr int W_SMEM_BYTES = WO_MISC + 16;                    // the dynamic shared memory must start on a 1024-byte boundary
static_assert(W_SMEM_BYTES <= 227 * 1024, "shared memory budget");

// TMEM columns (fp32): scores, state update, two output slots
constexpr uint32_t WT_P = 0, WT_U = 128, WT_O = 256, WT_P16 = 384, WT_COLS = 512;   // U and O are double buffered (64 columns each); P16: the masked scores as packed 16-bit pairs

// mbarrier indices
enum { B_FULL = 0, B_SFREE = 3, B_PREPPED = 6, B_PFULL = 9, B_PREADY = 10, B_STREADY = 11, B_UFULL = 12, B_OFULL = 14, B_OFREE = 16,
       B_PART = 18, B_XFREE = 20, B_STFREE = 22, B_OSTAGED = 23, B_COUNT = 25 };
static_assert(B_COUNT <= 32, "barrier slots");

struct WaveMaps { CUtensorMap q, k, v, gf, gb, o; };

struct WaveParams {
    BiglaParams p;
    uint32_t* ticket;      // [1]
    uint32_t* chain_cnt;   // [B*H][2]: state warps that have published step w (4 per step)
    uint32_t* chunk_flag;  // [B*H][nchunk]: raised by the first direction once its half of the chunk is in place
    float* mailbox;        // [B*H][2 dirs][2 slots][dk*dv + dk]
    int nseg, seg_chunks, nchunk;   // steps (work items) per chain, chunks per long step, chunks per sequence
    int n_long, short_chunks;       // the first n_long steps have seg_chunks chunks, the others short_chunks (the last one what is left)
    float inv_per_step, inv_H;   // reciprocals for the ticket decode (a division costs twenty-odd instructions)
};

// n / d and n % d for 0 <= n < 2^24 from a float reciprocal and two corrections.
__device__ __forceinline__ void divmod(int n, int d, float inv_d, int& q, int& r) {
    q = __float2int_rz(__int2float_rz(n) * inv_d);
    r = n - q * d;
    if (r >= d) { ++q; r -= d; }
    if (r < 0) { --q; r += d; }
}

struct Item { int bh, c0, dir, nch, w, b, h, pad; };   // c0: first chunk of the item (index into the sequence), nch: its chunks, w: its step


// Bounded wait on a global counter (one lane polls).
__device__ __forceinline__ void global_wait(const uint32_t* ctr, uint32_t need, volatile int* abort_flag) {
#pragma unroll 1
    for (uint32_t i = 0; i < (1u << 21); ++i) {
        if (ld_acquire_u32(ctr) >= need) return;
        if (*abort_flag) return;
        __nanosleep(64);
    }
    *abort_flag = 1;
}


// Operand scaling: a raw 16-bit pair times two fp32 scales.
template <typename T> struct ScalePair;
template <> struct ScalePair<__nv_bfloat16> {
    // bf16 has fp32's exponent range, so the scales themselves fit: round them to bf16 and multiply packed (two
    // roundings per operand element instead of one, no unpack / repack: the preparation warps are bound by issue slots)
    __device__ static uint32_t mul(uint32_t raw, float s0, float s1) {
        const __nv_bfloat162 sc = __floats2bfloat162_rn(s0, s1);
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&raw), sc);
        return *reinterpret_cast<const uint32_t*>(&r);
    }
};
template <> struct ScalePair<__half> {
    // fp16 cannot hold the scales (up to 2^115): product in fp32, one rounding
    __device__ static uint32_t mul(uint32_t raw, float s0, float s1) {
        const float2 f = Pack2<__half>::unpack(raw);
        return Pack2<__half>::pack(f.x * s0, f.y * s1);
    }
};

template <typename T, bool RAW, bool CLAMP, bool SO>
__global__ void __launch_bounds__(W_THREADS, 1) bigla_wave_kernel(const __grid_constant__ WaveMaps maps, const WaveParams wp) {
    const BiglaParams& p = wp.p;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {                                      // the swizzled tiles need it; never seen, but checked
        if (threadIdx.x == 0 && p.status) atomicOr(p.status, 1);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nseg = wp.nseg, seg_chunks = wp.seg_chunks;
    const int dir_first = (p.dir_mask & 1) ? 0 : 1, ndir = (p.dir_mask == 3) ? 2 : 1;
    const int per_step = p.B * p.H * ndir, total = per_step * nseg;
    // States-only call (no output tensor: the caller wants the chains' end states and summed log-gates, e.g. the summary pass
    // of the sequence split): q is not loaded, the scores, both output products, the masking and the staging are skipped;
    // what runs is the gate prefix, the K-tilde scaling, the state-update MMA and the state chain.
    constexpr bool so = SO;                                   // a template parameter: the full kernel carries none of this mode's code

    auto bar = [&](int i) { return sbase + WO_BAR + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + WO_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + WO_MISC + 4);
    volatile Item* ring = reinterpret_cast<volatile Item*>(smem + WO_ITEMS);
    float* vec = reinterpret_cast<float*>(smem + WO_VEC);
    const Waiter waiter{abort_flag, p.status};

    if (tid == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_SFREE + i), 1); mbar_init(bar(B_PREPPED + i), W_PREP_WARPS); }
        for (int i = 0; i < 2; ++i) mbar_init(bar(B_PART + i), W_PREP_WARPS);
        mbar_init(bar(B_XFREE), 1);
        mbar_init(bar(B_PFULL), 1); mbar_init(bar(B_PREADY), W_PREP_WARPS); mbar_init(bar(B_STREADY), 4); mbar_init(bar(B_STFREE), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_OFULL + i), 1); mbar_init(bar(B_OFREE + i), W_PREP_WARPS); mbar_init(bar(B_UFULL + i), 1); mbar_init(bar(B_OSTAGED + i), W_PREP_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(WT_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    auto read_item = [&](int idx, Item& it) {
        const volatile Item* r = ring + (idx & 7);
        it.bh = r->bh; it.c0 = r->c0; it.dir = r->dir; it.nch = r->nch; it.w = r->w;
    };
    // chunk (inside its segment) of sweep position ci, and its first token
    auto chunk_of = [&](const Item& it, int ci) { return it.dir ? it.nch - 1 - ci : ci; };
    auto state_zero = [&](const Item& it, int ci) { return ci == 0 && it.w == 0 && (it.dir ? p.init_b : p.init_f) == nullptr; };

    constexpr uint32_t IDESC_QK = make_idesc(Pack2<T>::FMT, 0, 0, 128, 128);
    constexpr uint32_t IDESC_OV = make_idesc(Pack2<T>::FMT, 0, 1, 128, 64);
    constexpr uint32_t IDESC_U = make_idesc(Pack2<T>::FMT, 1, 1, 64, 64);

    if (warp >= W_CTRL_WARP0) {
        // =============================== control warpgroup ===============================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(W_REGS_CTRL));
        if (tid == W_LOAD_WARP * 32) {
            // ---- load thread: work tickets and TMA loads, up to W_STAGES iterations ahead of the tensor core ----
            auto decode = [&](int t, Item& it) {               // ticket -> work item (nch = 0: no more work)
                it.nch = 0;
                if (t < total) {
                    int r;
                    divmod(t, per_step, wp.inv_per_step, it.w, r);
                    it.bh = ndir == 2 ? r >> 1 : r;
                    it.dir = dir_first + (ndir == 2 ? r & 1 : 0);
                    divmod(it.bh, p.H, wp.inv_H, it.b, it.h);
                    // steps of seg_chunks chunks, then shorter ones at the end of the scan (the last items of the
                    // schedule decide how evenly the SMs finish); a backward chain counts its chunks from the far end
                    int sc0, len;
                    if (it.w < wp.n_long) { sc0 = it.w * seg_chunks; len = seg_chunks; }
                    else { sc0 = wp.n_long * seg_chunks + (it.w - wp.n_long) * wp.short_chunks; len = min(wp.short_chunks, wp.nchunk - sc0); }
                    it.nch = len;
                    it.c0 = it.dir ? wp.nchunk - sc0 - len : sc0;
                }
            };
            // A ticket is drawn two items before its loads are issued and decoded one item before, when its value has long
            // arrived.  (Asking the next item's tiles into L2 at that point, with bulk prefetches, made the kernel 5 % slower:
            // the TMA unit and the memory system are loaded enough that the extra requests cost more than the latency they hide.)
            Item lcur, lnext;
            lcur.nch = 0; lcur.bh = lcur.c0 = lcur.dir = lcur.w = lcur.b = lcur.h = 0; lnext = lcur;
            int tk = (int)atomicAdd(wp.ticket, 1u);
            int l_items = -1, l_ci = 0;                        // the first pass through the item block only fills lnext
            #pragma unroll 1
            for (uint32_t lm = 0;; ++lm, ++l_ci) {
                while (l_ci == lcur.nch) {                     // next work item (twice at the start)
                    lcur = lnext;
                    if (l_items >= 0) {
                        volatile Item* r = ring + (l_items & 7);
                        r->bh = lcur.bh; r->c0 = lcur.c0; r->dir = lcur.dir; r->nch = lcur.nch; r->w = lcur.w; r->b = lcur.b; r->h = lcur.h;
                    }
                    ++l_items;
                    l_ci = 0;
                    decode(tk, lnext);                         // the item after this one
                    tk = (int)atomicAdd(wp.ticket, 1u);        // and the ticket of the one after that: consumed an item later
                    if (l_items > 0) break;                    // a real item is in lcur (an empty one ends the stream below)
                }
                const uint32_t s = lm % 3;
                if (lm >= 3) waiter.wait_lite(bar(B_SFREE + s), ((lm / 3) - 1) & 1);
                if (*abort_flag) break;
                if (lcur.nch == 0) { mbar_arrive_plain(bar(B_FULL + s)); break; }   // end marker: wakes the prep warps
                const int t0 = (lcur.c0 + chunk_of(lcur, l_ci)) * CHUNK;
                const int b = lcur.b, h = lcur.h;
                const uint32_t dst = sbase + s * W_STAGE_B, fb = bar(B_FULL + s);
                mbar_expect_tx(fb, so ? W_STAGE_B - W_TILE : W_STAGE_B);
                tma_load_4d(dst + WS_K, &maps.k, 0, t0, h, b, fb);
                tma_load_4d(dst + WS_G, lcur.dir ? &maps.gb : &maps.gf, 0, t0, h, b, fb);
                if (!so) tma_load_4d(dst + WS_Q, &maps.q, 0, t0, h, b, fb);
                tma_load_4d(dst + WS_V, &maps.v, 0, t0, h, b, fb);
            }
        } else if (warp == W_MMA_WARP) {
            // ---- MMA warp: all 32 lanes walk the loop (uniform control flow keeps the descriptor arithmetic in the
            // uniform datapath, off the issuing lane's critical path); lane 0 issues ----
            Item mcur; mcur.nch = 0; mcur.bh = mcur.c0 = mcur.dir = mcur.w = 0;
            int m_items = 0, m_ci = 0;
            const uint32_t st_lo = make_desc(sbase + WO_ST);
            #pragma unroll 1
            for (uint32_t m = 0;; ++m, ++m_ci) {
                const uint32_t s = m % 3, st = sbase + s * W_STAGE_B;
                waiter.wait_lite(bar(B_PREPPED + s), (m / 3) & 1);  // also orders the read of the work item after its write
                if (*abort_flag) break;
                if (m_ci == mcur.nch) { read_item(m_items, mcur); ++m_items; m_ci = 0; }
                if (mcur.nch == 0) break;
                // descriptor low words (16-byte units): +2 = 32 bytes along K inside a 128-byte row, +128 = 16 rows
                const uint32_t q_lo = make_desc(st + WS_Q), k_lo = make_desc(st + WS_K), v_lo = make_desc(st + WS_V);
                const uint32_t o_acc = tmem + WT_O + 64u * (m & 1u), u_acc = tmem + WT_U + 64u * (m & 1u);
                const bool s_zero = state_zero(mcur, m_ci);
                tc_fence_after();
                // The loops are walked by the whole warp and only the issuing instruction is predicated on the lane: the
                // control flow stays convergent, so loop counters and descriptor arithmetic run in the uniform datapath
                // instead of on the issuing lane (a lane-0 branch around the loops made every MMA cost ~150 cycles to issue).
                const bool issuer = lane == 0;
                if (so) {                                      // states only: the state update, then the stage is free
                    // the state warps' arrival for this iteration says they have taken the previous state update out of tensor
                    // memory: the update two back shared this one's slot and barrier (in a full call the wait before step (b) is
                    // what keeps the MMA warp from running ahead)
                    waiter.wait_lite(bar(B_STREADY), m & 1);
                    tc_fence_after();
#pragma unroll
                    for (uint32_t k8 = 0; k8 < CHUNK / 16; ++k8) { if (issuer) tc_mma(u_acc, k_lo + 128 * k8, v_lo + 128 * k8, IDESC_U, k8 > 0); }
                    if (issuer) { tc_commit(bar(B_UFULL + (m & 1u))); tc_commit(bar(B_SFREE + s)); }
                    __syncwarp();
                    continue;
                }
                // the barriers of (b) are asked about before (a) and the state update are issued, that of (c) before (b)
                const uint32_t pre_st = mbar_test_wait(bar(B_STREADY), m & 1);
                const uint32_t pre_of = m >= 2 ? mbar_test_wait(bar(B_OFREE + (m & 1)), ((m >> 1) - 1) & 1) : 1u;
                // (a) scores, and right behind them the state update: it needs only the prepared tiles, and the
                // state chain -- the one sequential dependency of the kernel -- waits for nothing else
#pragma unroll
                for (uint32_t k4 = 0; k4 < WDK / 16; ++k4) { if (issuer) tc_mma(tmem + WT_P, q_lo + 2 * k4, k_lo + 2 * k4, IDESC_QK, k4 > 0); }
                if (issuer) tc_commit(bar(B_PFULL));
#pragma unroll
                for (uint32_t k8 = 0; k8 < CHUNK / 16; ++k8) { if (issuer) tc_mma(u_acc, k_lo + 128 * k8, v_lo + 128 * k8, IDESC_U, k8 > 0); }
                if (issuer) tc_commit(bar(B_UFULL + (m & 1u)));
                // (b) product with the entering state
                if (!pre_st) waiter.wait_lite(bar(B_STREADY), m & 1);
                if (!pre_of) waiter.wait_lite(bar(B_OFREE + (m & 1)), ((m >> 1) - 1) & 1);
                const uint32_t pre_pr = mbar_test_wait(bar(B_PREADY), m & 1);
                tc_fence_after();
                if (!s_zero) {
#pragma unroll
                    for (uint32_t k4 = 0; k4 < WDK / 16; ++k4) { if (issuer) tc_mma(o_acc, q_lo + 2 * k4, st_lo + 128 * k4, IDESC_OV, k4 > 0); }
                }
                if (issuer) tc_commit(bar(B_STFREE));          // the state operand may be overwritten
                // (c) masked scores x v
                if (!pre_pr) waiter.wait_lite(bar(B_PREADY), m & 1);
                tc_fence_after();
#pragma unroll
                for (uint32_t k8 = 0; k8 < CHUNK / 16; ++k8) {      // A = masked scores in tensor memory, 8 packed columns per K = 16 step
                    if (issuer) tc_mma_ts(o_acc, tmem + WT_P16 + 8 * k8, v_lo + 128 * k8, IDESC_OV, !s_zero || k8 > 0);
                }
                if (issuer) { tc_commit(bar(B_OFULL + (m & 1))); tc_commit(bar(B_SFREE + s)); }
                __syncwarp();
            }
        } else if (tid == W_STORE_WARP * 32) {
            // ---- store thread: the output tile of iteration j, staged by the score warps, goes out as one TMA store (first direction to reach the chunk) or one TMA reduction (second).
            // The global-memory latencies of the hand-over between the directions (write complete -> flag; flag -> add)
            // are spent here, by a thread that has nothing else to do.
            Item cur; cur.nch = 0; cur.bh = cur.c0 = cur.dir = cur.w = 0;
            int items = 0, ci = 0;
            #pragma unroll 1
            for (uint32_t j = 0; !so; ++j, ++ci) {              // (a states-only call stages nothing)
                waiter.wait_lite(bar(B_OSTAGED + (j & 1)), (j >> 1) & 1);
                if (*abort_flag) break;
                if (ci == cur.nch) { read_item(items, cur); cur.b = ring[items & 7].b; cur.h = ring[items & 7].h; ++items; ci = 0; }
                if (cur.nch == 0) break;
                const int c = chunk_of(cur, ci);
                const int t0 = (cur.c0 + c) * CHUNK, b = cur.b, h = cur.h;
                // the step at which the other direction reaches this chunk: it counts chunks from the other end of the
                // sequence, through the same schedule of long steps followed by short ones
                const int sc_other = cur.dir ? cur.c0 + c : wp.nchunk - 1 - (cur.c0 + c);
                const int n_long_chunks = wp.n_long * seg_chunks;
                const int w_other = sc_other < n_long_chunks ? sc_other / seg_chunks : wp.n_long + (sc_other - n_long_chunks) / wp.short_chunks;
                // Which direction stores and which adds is fixed by the schedule: the one whose step is earlier; within the
                // same step the one that reaches the chunk earlier inside its item (so neither item starts by waiting for the
                // other: short sequences are one step); on a full tie the forward one.
                const int pos_mine = ci, pos_other = (sc_other < n_long_chunks ? sc_other % seg_chunks : (sc_other - n_long_chunks) % wp.short_chunks);
                const bool first = ndir == 1 || cur.w < w_other ||
                                   (cur.w == w_other && (pos_mine < pos_other || (pos_mine == pos_other && cur.dir == 0)));
                uint32_t* flag = wp.chunk_flag + (size_t)cur.bh * wp.nchunk + cur.c0 + c;   // one flag per chunk of the sequence
                const uint32_t src = sbase + WO_X;
                if (first) {
                    tma_store_4d(&maps.o, 0, t0, h, b, src);     // rows past L are clipped by the tensor map
                } else {
                    global_wait(flag, 1u, abort_flag); // the other direction's half must be in place
                    tma_reduce_add_4d(&maps.o, 0, t0, h, b, src);
                }
                bulk_commit();
                bulk_store_wait_read();
                mbar_arrive_plain(bar(B_XFREE));                 // the tile may take the next iteration's scores
                if (first && ndir == 2) {                      // publish my half of the chunk once it is written
                    bulk_store_wait_all();
                    __threadfence();
                    atomicAdd(flag, 1u);
                }
            }
            bulk_store_wait_all();
        }
    } else if (warp < W_PREP_WARPS) {
        // =============================== prep warps: gates and operand scaling, in place ===============================
        // A warp owns 8 tokens (one group), a half-warp 4 consecutive scan positions, a lane 4 channels of them
        // (8-byte shared-memory accesses: a half-warp covers one 128-byte token row).  Scan position sp = 4*half + u is
        // token 8*warp + (sp ^ dmask): the same code serves both directions.  Gate form (raw logits or log-gates) and the
        // lower clamp are template parameters: the token loops carry no branch, so their 16 elements overlap.
        const int grp = warp;
        const float coef = RAW ? -1.f / p.gate_norm : LOG2E;  // log2-gate = coef * (RAW ? log2(1 + 2^(-x log2 e)) : x)
        const float clamp_lo = CLAMP ? p.clamp_min * LOG2E : -INFINITY;
        const int half = lane >> 4, c4l = lane & 15;          // my half of the group, my 4 channels: 4*c4l .. 4*c4l+3
        const uint32_t sw_in = (uint32_t)(c4l & 1) * 8, chunk = (uint32_t)c4l >> 1;
        // The same warps mask the scores of the iteration before and stage the output of the one before that (a warp owns
        // the 32 query rows of its TMEM lane quadrant and a quarter of the columns): by the time a trip reaches them the
        // tensor core has long finished what they need, sixteen warps share work that four would serialise, and the SM
        // runs one big instruction stream instead of two.
        const int quad = warp & 3, sub = warp >> 2;           // my TMEM lane quadrant; my quarter of the key blocks / output columns
        const int row = 32 * quad + lane;
        const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
        const float o_sign = p.qscale;                        // scale * out_scale, applied to the finished accumulators
        Item cur; cur.nch = 0; cur.bh = cur.c0 = cur.dir = cur.w = 0;
        int items = 0, ci = -1, dir_prev = 0;
        bool ended = false;
        uint32_t end_m = 0;                                   // first iteration that does not exist
        #pragma unroll 1
        for (uint32_t m = 0;; ++m) {
            const uint32_t s = m % 3;
            bool have = false;
            const int dir_mask_it = dir_prev;                 // direction of iteration m - 1 (the one whose scores are masked in this trip)
            float4 gl[4];                                     // cumulative log2-gates of my 4 tokens, from the group's first token
            uint8_t* stg = smem + s * W_STAGE_B;
            int dmask = 0;
            // A test of an mbarrier costs a few hundred cycles even when its phase completed long ago (it queues behind the
            // CTA's shared-memory traffic).  The barriers this trip will need are therefore all asked about here, at once and
            // without blocking; the answers arrive during the gate phase, and a wait loop is entered later only on "not yet".
            uint32_t pre_pfull = 0, pre_ofull = 0, pre_xfree = 0;
            if (m >= 1) pre_pfull = mbar_test_wait(bar(B_PFULL), (m - 1) & 1);
            if (m >= 2) pre_ofull = mbar_test_wait(bar(B_OFULL + (m & 1)), ((m - 2) >> 1) & 1);
            if (m >= 3) pre_xfree = mbar_test_wait(bar(B_XFREE), (m - 3) & 1);
            if (!ended) {
            waiter.wait_lite(bar(B_FULL + s), (m / 3) & 1);
            __syncwarp();
            if (*abort_flag) break;
            ++ci;
            if (ci == cur.nch || cur.nch == 0) { read_item(items, cur); ++items; ci = 0; }
            if (cur.nch == 0) {                               // end marker: pass it on to the MMA warp and the state warps
                if (lane == 0) mbar_arrive_plain(bar(B_PREPPED + s));
                ended = true; end_m = m;
            } else {
            have = true;
            dir_prev = cur.dir;
            const int t0 = (cur.c0 + chunk_of(cur, ci)) * CHUNK;
            const int n_valid = p.L - t0;                     // rows at or past it are padding: decay 1
            dmask = cur.dir ? 7 : 0;
            // ---- gate phase: transform, running sums over my 4 tokens, group sum published ----
            {
                uint2 raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    raw[u] = *reinterpret_cast<const uint2*>(stg + WS_G + (grp * 8 + ((half * 4 + u) ^ dmask)) * 128 + c4l * 8);
                float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 a = Pack2<T>::unpack(raw[u].x), b2 = Pack2<T>::unpack(raw[u].y);
                    float4 t = make_float4(a.x, a.y, b2.x, b2.y);
                    if (RAW) {                                // log2(1 + 2^(-x log2 e)) = -log2 sigmoid(x)
                        const F2 nl = f2_make(-LOG2E, -LOG2E), one = f2_make(1.f, 1.f);
                        const F2 y01 = f2_mul(f2_make(t.x, t.y), nl), y23 = f2_mul(f2_make(t.z, t.w), nl);
                        const F2 e01 = f2_add(one, f2_make(ex2(f2_lo(y01)), ex2(f2_hi(y01)))), e23 = f2_add(one, f2_make(ex2(f2_lo(y23)), ex2(f2_hi(y23))));
                        t.x = lg2(f2_lo(e01)); t.y = lg2(f2_hi(e01)); t.z = lg2(f2_lo(e23)); t.w = lg2(f2_hi(e23));
                    }
                    const float cu = grp * 8 + ((half * 4 + u) ^ dmask) < n_valid ? coef : 0.f;   // padding rows: gate 0
                    if (CLAMP) {
                        run.x += fmaxf(t.x * cu, clamp_lo); run.y += fmaxf(t.y * cu, clamp_lo);
                        run.z += fmaxf(t.z * cu, clamp_lo); run.w += fmaxf(t.w * cu, clamp_lo);
                    } else {
                        const F2 c2 = f2_make(cu, cu);
                        const F2 r01 = f2_fma(f2_make(t.x, t.y), c2, f2_make(run.x, run.y)), r23 = f2_fma(f2_make(t.z, t.w), c2, f2_make(run.z, run.w));
                        run = make_float4(f2_lo(r01), f2_hi(r01), f2_lo(r23), f2_hi(r23));
                    }
                    gl[u] = run;
                }
                // the second half-warp continues the first half-warp's sum; it also knows the group's total
                float4 first;
                first.x = __shfl_sync(0xffffffffu, run.x, c4l); first.y = __shfl_sync(0xffffffffu, run.y, c4l);
                first.z = __shfl_sync(0xffffffffu, run.z, c4l); first.w = __shfl_sync(0xffffffffu, run.w, c4l);
                float* part = reinterpret_cast<float*>(smem + WO_PART) + (m & 1) * (W_PREP_WARPS * WDK);
                if (half) {
                    reinterpret_cast<float4*>(part)[grp * 16 + c4l] = make_float4(run.x + first.x, run.y + first.y, run.z + first.z, run.w + first.w);
#pragma unroll
                    for (int u = 0; u < 4; ++u) { gl[u].x += first.x; gl[u].y += first.y; gl[u].z += first.z; gl[u].w += first.w; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive_plain(bar(B_PART + (m & 1)));
            }
            }
            }
            // ---- scores of iteration j = m - 1: TMEM -> masked 16-bit tiles (my 32 rows x key block `sub`) ----
            if (!so && m >= 1 && (!ended || m - 1 < end_m)) {
                const uint32_t j = m - 1;
                if (!pre_pfull) waiter.wait_lite(bar(B_PFULL), j & 1);
                __syncwarp();
                if (*abort_flag) break;
                tc_fence_after();
                const int cb = sub, dir = dir_mask_it;
                // The masked scores go back to tensor memory as packed 16-bit pairs (64 columns for 128 keys) and step (c)
                // reads its A operand from there: no shared-memory tile, no proxy fence, and no wait for the state update to
                // have read the k tile.  The slot is single: step (c) of iteration j-1 has completed before the scores of
                // iteration j exist (its commit precedes theirs in the MMA warp's program order).
                // A 32x32 block of scores is wholly kept, wholly masked, or on the diagonal (warp-uniform test)
                const bool all_zero = dir ? cb < quad : cb > quad;
                uint32_t pk[16];
                if (all_zero) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = 0u;
                } else {
                    float a[32];
                    tc_ld32(tmem + lane_base + WT_P + 32 * cb, a);
                    tc_wait_ld();
                    if (cb == quad) {                                     // the diagonal block: bit e says whether key e is kept for my row
                        const uint32_t keep = dir ? ~((1u << lane) - 1u) : (lane == 31 ? 0xffffffffu : (2u << lane) - 1u);
#pragma unroll
                        for (int e = 0; e < 32; ++e) a[e] = (keep >> e) & 1u ? a[e] : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = Pack2<T>::pack(a[2 * i], a[2 * i + 1]);
                }
                tc_st16(tmem + lane_base + WT_P16 + 16 * cb, pk);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_plain(bar(B_PREADY));
            }
            // ---- output of iteration j = m - 2: accumulator slot -> 16-bit staging tile (my 32 rows x 16 columns) ----
            if (!so && m >= 2 && (!ended || m - 2 < end_m)) {
                const uint32_t j = m - 2;
                if (!pre_ofull) waiter.wait_lite(bar(B_OFULL + (j & 1)), (j >> 1) & 1);
                if (j > 0 && !pre_xfree) waiter.wait_lite(bar(B_XFREE), (j - 1) & 1);        // the store thread has sent the previous tile
                __syncwarp();
                if (*abort_flag) break;
                tc_fence_after();
                float a[16];
                tc_ld16(tmem + lane_base + WT_O + 64u * (j & 1u) + 16 * sub, a);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_plain(bar(B_OFREE + (j & 1)));   // the slot is read: hand it back
                uint8_t* orow = smem + WO_X + row * 128;
                const F2 os2 = f2_make(o_sign, o_sign);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t w[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const F2 v = f2_mul(os2, f2_make(a[8 * i + 2 * k], a[8 * i + 2 * k + 1]));
                        w[k] = Pack2<T>::pack(f2_lo(v), f2_hi(v));
                    }
                    *reinterpret_cast<uint4*>(orow + (((uint32_t)(2 * sub + i) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive_plain(bar(B_OSTAGED + (j & 1)));
            }
            // ---- second half of the preparation of iteration m: by now the other warps' group sums are in (the masking and
            // staging above ran while they arrived), so the wait below is a formality ----
            if (have) {
            // raw operand rows into registers
            uint2 rk[4], rq[4];
            uint32_t offs[4];
            const uint32_t pre_part = mbar_test_wait(bar(B_PART + (m & 1)), (m >> 1) & 1);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t r7 = (uint32_t)((half * 4 + u) ^ dmask);
                offs[u] = (uint32_t)(grp * 8 + r7) * 128 + ((chunk ^ r7) << 4) + sw_in;
                rk[u] = *reinterpret_cast<const uint2*>(stg + WS_K + offs[u]);
                rq[u] = so ? make_uint2(0u, 0u) : *reinterpret_cast<const uint2*>(stg + WS_Q + offs[u]);
            }
            if (!pre_part) waiter.wait_lite(bar(B_PART + (m & 1)), (m >> 1) & 1);     // all sixteen group sums are in
            __syncwarp();
            if (*abort_flag) break;
            // ---- my group's offset: (sum of the groups scanned before mine) - G_ref, G_ref = sum of the first 8 groups in
            // scan order.  Half-warp gq reads groups 8 gq .. 8 gq + 7 (scan order) for its 4 channels; one exchange. ----
            float4 off;
            {
                const float4* part = reinterpret_cast<const float4*>(smem + WO_PART) + (m & 1) * (W_PREP_WARPS * 16) + c4l;
                const int flip = cur.dir ? W_PREP_WARPS - 1 : 0;          // scan position go <-> group go ^ flip
                const int mygo = grp ^ flip;
                // two-wide fp32 arithmetic (the workers are bound by instruction issue)
                F2 s01 = f2_make(0.f, 0.f), s23 = s01, b01 = s01, b23 = s01;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int go = half * 8 + i;
                    const float4 t = part[(go ^ flip) * 16];
                    const F2 t01 = f2_make(t.x, t.y), t23 = f2_make(t.z, t.w);
                    s01 = f2_add(s01, t01); s23 = f2_add(s23, t23);
                    const float k = go < mygo ? 1.f : 0.f;
                    const F2 kk = f2_make(k, k);
                    b01 = f2_fma(kk, t01, b01); b23 = f2_fma(kk, t23, b23);
                }
                const float4 sum = make_float4(f2_lo(s01), f2_hi(s01), f2_lo(s23), f2_hi(s23));
                const float4 bef = make_float4(f2_lo(b01), f2_hi(b01), f2_lo(b23), f2_hi(b23));
                float4 osum, obef;
                osum.x = __shfl_xor_sync(0xffffffffu, sum.x, 16); osum.y = __shfl_xor_sync(0xffffffffu, sum.y, 16);
                osum.z = __shfl_xor_sync(0xffffffffu, sum.z, 16); osum.w = __shfl_xor_sync(0xffffffffu, sum.w, 16);
                obef.x = __shfl_xor_sync(0xffffffffu, bef.x, 16); obef.y = __shfl_xor_sync(0xffffffffu, bef.y, 16);
                obef.z = __shfl_xor_sync(0xffffffffu, bef.z, 16); obef.w = __shfl_xor_sync(0xffffffffu, bef.w, 16);
                const float4 gref = half ? osum : sum;                    // the half-warp that read the first 8 groups has it
                off = make_float4(bef.x + obef.x - gref.x, bef.y + obef.y - gref.y, bef.z + obef.z - gref.z, bef.w + obef.w - gref.w);
                if (grp == 0 && half == 0) {                              // [G_ref | G_last] of this iteration for the state warps
                    float4* ve = reinterpret_cast<float4*>(vec + (m & 3) * 128) + c4l;
                    ve[0] = gref;
                    ve[16] = make_float4(sum.x + osum.x, sum.y + osum.y, sum.z + osum.z, sum.w + osum.w);
                }
            }
            // ---- scale phase ----
            // Log-gates are <= 0, so a lane's exponents are monotone along its 4 tokens: the largest magnitude is at one
            // of the two ends.  Beyond the range the factorisation covers, exponents are clamped and the call is flagged.
            float worst = fmaxf(fmaxf(fabsf(off.x + gl[0].x), fabsf(off.y + gl[0].y)), fmaxf(fabsf(off.z + gl[0].z), fabsf(off.w + gl[0].w)));
            worst = fmaxf(worst, fmaxf(fmaxf(fabsf(off.x + gl[3].x), fabsf(off.y + gl[3].y)), fmaxf(fabsf(off.z + gl[3].z), fabsf(off.w + gl[3].w))));
            const bool out_of_range = __any_sync(0xffffffffu, !(worst <= MAX_EXPONENT2));
            if (out_of_range) {                               // rare: clamp in place, flag the call
                if (lane == 0 && p.status) atomicOr(p.status, 2);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    gl[u].x = fminf(fmaxf(off.x + gl[u].x, -MAX_EXPONENT2), MAX_EXPONENT2) - off.x;
                    gl[u].y = fminf(fmaxf(off.y + gl[u].y, -MAX_EXPONENT2), MAX_EXPONENT2) - off.y;
                    gl[u].z = fminf(fmaxf(off.z + gl[u].z, -MAX_EXPONENT2), MAX_EXPONENT2) - off.z;
                    gl[u].w = fminf(fmaxf(off.w + gl[u].w, -MAX_EXPONENT2), MAX_EXPONENT2) - off.w;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float ex = off.x + gl[u].x, ey = off.y + gl[u].y, ez = off.z + gl[u].z, ew = off.w + gl[u].w;
                uint2 ko, qo;                                 // scale * out_scale is applied to the output instead
                ko.x = ScalePair<T>::mul(rk[u].x, ex2(-ex), ex2(-ey)); ko.y = ScalePair<T>::mul(rk[u].y, ex2(-ez), ex2(-ew));
                if (!so) { qo.x = ScalePair<T>::mul(rq[u].x, ex2(ex), ex2(ey)); qo.y = ScalePair<T>::mul(rq[u].y, ex2(ez), ex2(ew)); }
                *reinterpret_cast<uint2*>(stg + WS_K + offs[u]) = ko;
                if (!so) *reinterpret_cast<uint2*>(stg + WS_Q + offs[u]) = qo;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar(B_PREPPED + s));
            }
            if (ended && (so || m >= end_m + 1)) {            // everything that exists is masked and staged: tell the store thread
                if (lane == 0 && !so) mbar_arrive_plain(bar(B_OSTAGED + (end_m & 1)));
                break;
            }
        }
    } else if (warp < W_CTRL_WARP0) {
        // =============================== state warps ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(W_REGS_STATE));
        const int quad = warp & 3;
        const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
        const int st_row = 16 * quad + (lane & 15);           // key channel: an M=64 accumulator puts row r in lane (r%16) + 32*(r/16)
        const int hi = lane >> 4;                             // lanes 16-31 take columns 16..31 and 48..63 of the same rows
        auto col_of = [&](int j) { return 32 * (j >> 4) + 16 * hi + (j & 15); };
        constexpr int NE = WDK * WDV, SLOT = NE + WDK;
        float S[32];
        float gacc = 0.f;                                     // summed log2-gates of my channel along the chain so far
        Item cur; cur.nch = 0; cur.bh = cur.c0 = cur.dir = cur.w = 0;
        int items = 0, ci = 0;
        bool s_zero = true;
        #pragma unroll 1
        for (uint32_t m = 0;; ++m, ++ci) {
            const uint32_t s = m % 3;
            // The work item is known as soon as its loads are under way: the state entering a new segment is fetched
            // from the mailbox while the prep warps still work on the iteration (two trips to L2 that would otherwise
            // sit in front of the state product).
            waiter.wait_lite(bar(B_FULL + s), (m / 3) & 1);
            __syncwarp();
            if (*abort_flag) break;
            if (ci == cur.nch) { read_item(items, cur); ++items; ci = 0; }
            if (cur.nch == 0) break;
            if (ci == 0) {                                    // the chain enters a new segment
                const float* src = nullptr;
                if (cur.w == 0) {
                    // the caller's states are [dk, dv] per (b, h): with dk = 32 the kernel's upper 32 key channels are padding
                    const float* init = cur.dir ? p.init_b : p.init_f;
                    if (init) src = init + (size_t)cur.bh * p.dk * WDV;
                    gacc = 0.f;
                } else {
                    uint32_t* cnt = wp.chain_cnt + cur.bh * 2 + cur.dir;
                    global_wait(cnt, 4u * (uint32_t)cur.w, abort_flag);     // taken by the whole warp, like every wait here
                    const float* box = wp.mailbox + (((size_t)cur.bh * 2 + cur.dir) * 2 + ((cur.w - 1) & 1)) * SLOT;
                    src = box;
                    gacc = __ldcg(box + NE + st_row);
                }
                s_zero = src == nullptr;
                const bool row_in = cur.w > 0 || st_row < p.dk;     // (the mailbox holds all 64 rows, the padding ones zero)
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 t4 = src && row_in ? __ldcg(reinterpret_cast<const float4*>(src + st_row * WDV + col_of(j))) : make_float4(0.f, 0.f, 0.f, 0.f);
                    S[j] = t4.x; S[j + 1] = t4.y; S[j + 2] = t4.z; S[j + 3] = t4.w;
                }
            }
            waiter.wait_lite(bar(B_PREPPED + s), (m / 3) & 1);   // G_ref, G_last of this iteration are written
            __syncwarp();
            if (*abort_flag) break;
            const float* ve = vec + (m & 3) * 128;             // [G_ref | G_last] of this iteration, log2 units
            if (m > 0 && !so) {                               // the previous iteration's state product has read the operand
                waiter.wait_lite(bar(B_STFREE), (m - 1) & 1);
                __syncwarp();
            }
            if (!s_zero && !so) {                             // bf16(2^G_ref * S_in), MN-major [channel][value]
                const float eg = ex2(ve[st_row]);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 w4;
                    w4.x = Pack2<T>::pack(S[j] * eg, S[j + 1] * eg); w4.y = Pack2<T>::pack(S[j + 2] * eg, S[j + 3] * eg);
                    w4.z = Pack2<T>::pack(S[j + 4] * eg, S[j + 5] * eg); w4.w = Pack2<T>::pack(S[j + 6] * eg, S[j + 7] * eg);
                    *reinterpret_cast<uint4*>(smem + WO_ST + swz(st_row, col_of(j) * 2)) = w4;
                }
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar(B_STREADY));
            waiter.wait_lite(bar(B_UFULL + (m & 1)), (m >> 1) & 1);
            __syncwarp();
            tc_fence_after();
            {
                const float g_ref = ve[st_row], g_last = ve[64 + st_row];
                const float e_last = ex2(g_last), e_rel = ex2(g_last - g_ref);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float u[32];
                    tc_ld32(tmem + lane_base + WT_U + 64u * (m & 1u) + 32 * half, u);   // rows live in lanes 0-15 of the warp
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float up = __shfl_sync(0xffffffffu, u[16 + j], lane & 15);   // columns 16-31 go to lanes 16-31
                        const float mine = hi ? up : u[j];
                        S[16 * half + j] = fmaf(S[16 * half + j], e_last, e_rel * mine);
                    }
                }
                gacc += g_last;
            }
            tc_fence_before();
            s_zero = false;
            if (ci == cur.nch - 1) {                          // the chain leaves the segment: mailbox, or the caller's outputs
                const bool last = cur.w == nseg - 1;
                float* dst = nullptr;
                float* gdst = nullptr;
                if (last) {
                    float* fin = cur.dir ? p.final_b : p.final_f;
                    float* ld = cur.dir ? p.logdecay_b : p.logdecay_f;
                    if (fin) dst = fin + (size_t)cur.bh * p.dk * WDV;
                    if (ld) gdst = ld + (size_t)cur.bh * p.dk;
                } else {
                    float* box = wp.mailbox + (((size_t)cur.bh * 2 + cur.dir) * 2 + (cur.w & 1)) * SLOT;
                    dst = box; gdst = box + NE;
                }
                const bool row_out = !last || st_row < p.dk;        // the caller's tensors end at dk rows
                if (dst && row_out) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(dst + st_row * WDV + col_of(j)) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
                }
                if (gdst && hi == 0 && row_out) gdst[st_row] = last ? gacc * LN2 : gacc;   // the caller gets natural-log units
                if (!last) {
                    __syncwarp();
                    if (lane == 0) { __threadfence(); atomicAdd(wp.chain_cnt + cur.bh * 2 + cur.dir, 1u); }
                }
            }
        }
    }
    // ---- teardown: every role has left its loop; all MMAs were waited for by their consumers ----
    tc_fence_before();
    __syncthreads();
    if (tid == 32 && *abort_flag && p.status) atomicOr(p.status, 1);   // a bounded wait ran out somewhere in this CTA
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(WT_COLS) : "memory");
    }
}

size_t wave_counter_bytes(int B, int H, int L) {       // ticket, two progress counters per (b, h), one flag per chunk
    return ((1 + 2 * (size_t)B * H + (size_t)B * H * ((L + CHUNK - 1) / CHUNK)) * sizeof(uint32_t) + 255) & ~(size_t)255;
}

int wave_sm_count() {
    static int sm_count[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (!sm_count[dev]) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        sm_count[dev] = sms;
    }
    return sm_count[dev];
}

// Chunks per work item: the longest of 8, 4, 2 that still leaves two segments per sequence and about six items per SM
int wave_seg_chunks(const BiglaParams& p, int sms) {
    const long long chains = (long long)p.B * p.H * (p.dir_mask == 3 ? 2 : 1);
    int sc = W_SEG_CHUNKS_MAX;
    while (sc > W_SEG_CHUNKS_MIN) {
        const int nseg = (p.L + sc * CHUNK - 1) / (sc * CHUNK);
        if (nseg >= 2 && chains * nseg >= 6ll * sms) break;
        sc /= 2;
    }
    return sc;
}

template <typename T, bool RAW, bool CLAMP, bool SO>
int launch_wave(const BiglaParams& p, const WaveMaps& maps, void* ws, cudaStream_t stream) {
    const int sms = wave_sm_count();
    if (sms <= 0) return VIG_ERR_DEVICE;
    const int seg_chunks = wave_seg_chunks(p, sms);
    const int nchunk = (p.L + CHUNK - 1) / CHUNK;
    // the schedule ends with half-length steps: the tail of the ticket queue then has items half as long, and the SMs finish
    // within half an item of each other
    const int short_chunks = seg_chunks >= 4 ? seg_chunks / 2 : seg_chunks;
    const int n_long = short_chunks == seg_chunks ? 0 : (nchunk / seg_chunks > 1 ? nchunk / seg_chunks - 1 : 0);
    const int nseg = n_long + (nchunk - n_long * seg_chunks + short_chunks - 1) / short_chunks;
    const int BH = p.B * p.H;
    WaveParams wp;
    wp.p = p;
    wp.nseg = nseg;
    wp.seg_chunks = seg_chunks;
    wp.nchunk = nchunk;
    wp.n_long = n_long;
    wp.short_chunks = short_chunks;
    wp.inv_per_step = 1.0f / (float)(BH * (p.dir_mask == 3 ? 2 : 1));
    wp.inv_H = 1.0f / (float)p.H;
    wp.ticket = reinterpret_cast<uint32_t*>(ws);
    wp.chain_cnt = wp.ticket + 1;
    wp.chunk_flag = wp.chain_cnt + 2 * (size_t)BH;
    const size_t cb = wave_counter_bytes(p.B, p.H, p.L);
    wp.mailbox = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + cb);
    cudaError_t e;
    if ((e = cudaMemsetAsync(ws, 0, cb, stream)) != cudaSuccess) return (int)e;
    auto kern = bigla_wave_kernel<T, RAW, CLAMP, SO>;
    if ((e = ensure_smem_attr(reinterpret_cast<const void*>(kern), W_SMEM_BYTES)) != cudaSuccess) return (int)e;
    const int ndir = p.dir_mask == 3 ? 2 : 1;
    const long long items = (long long)BH * ndir * nseg;
    const int grid = (int)(items < sms ? items : sms);
    kern<<<grid, W_THREADS, W_SMEM_BYTES, stream>>>(maps, wp);
    return (int)cudaGetLastError();
}

}  // namespace

bool bigla_wave_supported(const BiglaParams& p) {
    if (p.dtype != VIG_DTYPE_BF16 && p.dtype != VIG_DTYPE_F16) return false;
    // dk = 32 runs as dk = 64 with the upper 32 key channels zero: the q / k / gate boxes are declared 64 wide over tensors
    // of 32 channels and the TMA unit fills the rest with zeros, which stay zero through the scaling; half of the MMA
    // work on those operands is wasted, the DRAM traffic is that of dk = 32
    if (p.dv != WDV || (p.dk != WDK && p.dk != 32) || p.B * p.H < 1 || p.L < 1) return false;
    if (p.o ? !p.q : !(p.final_f || p.final_b || p.logdecay_f || p.logdecay_b)) return false;   // an output, or a states-only call
    if (p.dir_mask < 1 || p.dir_mask > 3) return false;
    if ((long long)p.B * p.H * 2 * ((p.L + W_SEG_CHUNKS_MIN * CHUNK - 1) / (W_SEG_CHUNKS_MIN * CHUNK)) >= (1ll << 24)) return false;   // tickets are decoded in fp32
    if ((p.o && !tc::tma_ok(p.q, p.sq, p.B, p.H)) || !tc::tma_ok(p.k, p.sk, p.B, p.H) || !tc::tma_ok(p.v, p.sv, p.B, p.H)) return false;
    if ((p.dir_mask & 1) && (!p.gf || !tc::tma_ok(p.gf, p.sgf, p.B, p.H))) return false;
    if ((p.dir_mask & 2) && (!p.gb || !tc::tma_ok(p.gb, p.sgb, p.B, p.H))) return false;
    if (p.o && ((reinterpret_cast<uintptr_t>(p.o) & 15) || (p.so[0] * 2) % 16 || (p.so[1] * 2) % 16 || (p.so[2] * 2) % 16)) return false;
    return tc::encode_fn() != nullptr;
}

// Measured on B200: with at least as many (sequence, direction) chains as SMs and two or more segments per sequence the
// wavefront form beats the segment-parallel forms (0.46 against 0.58 ms at 64 x 3 sequences of 4096 tokens); with
// fewer chains its CTAs idle, and a single segment has nothing to hand on.
bool bigla_wave_preferred(const BiglaParams& p) {
    const int sms = wave_sm_count();
    const int ndir = p.dir_mask == 3 ? 2 : 1;
    return sms > 0 && p.L > W_SEG_CHUNKS_MIN * CHUNK && (long long)p.B * p.H * ndir >= sms;
}

// Counters (ticket, chain progress, chunk flags) followed by the state mailboxes.
size_t bigla_wave_workspace(int B, int H, int L, int dk, int dv) {
    (void)dk; (void)dv;                                     // the mailbox slots hold the kernel's 64 x 64 states whatever dk is
    return wave_counter_bytes(B, H, L) + (size_t)B * H * 2 * 2 * ((size_t)WDK * WDV + WDK) * sizeof(float);
}

int bigla_wave_launch(const BiglaParams& p, void* ws, size_t ws_bytes, cudaStream_t stream) {
    if (!ws || ws_bytes < bigla_wave_workspace(p.B, p.H, p.L, p.dk, p.dv)) return VIG_ERR_WORKSPACE;
    WaveMaps maps;
    const void* gfs = p.gf ? p.gf : p.gb;
    const int64_t* gfst = p.gf ? p.sgf : p.sgb;
    const void* gbs = p.gb ? p.gb : p.gf;
    const int64_t* gbst = p.gb ? p.sgb : p.sgf;
    // a states-only call reads no q and writes no output: those two maps stand in with the k / v tensors and are never used
    const bool so = p.o == nullptr;
    if (!tc::make_map(&maps.q, so ? p.k : p.q, so ? p.sk : p.sq, p.B, p.H, p.L, p.dk, p.dtype, true, WDK) ||
        !tc::make_map(&maps.k, p.k, p.sk, p.B, p.H, p.L, p.dk, p.dtype, true, WDK) ||
        !tc::make_map(&maps.v, p.v, p.sv, p.B, p.H, p.L, p.dv, p.dtype, true) ||
        !tc::make_map(&maps.gf, gfs, gfst, p.B, p.H, p.L, p.dk, p.dtype, false, WDK) ||
        !tc::make_map(&maps.gb, gbs, gbst, p.B, p.H, p.L, p.dk, p.dtype, false, WDK) ||
        !tc::make_map(&maps.o, so ? p.v : p.o, so ? p.sv : p.so, p.B, p.H, p.L, p.dv, p.dtype, true))
        return VIG_ERR_DEVICE;
    // gate form and clamp are compile-time properties of the kernel: no branch inside its token loops
    const bool raw = p.gate_norm > 0.f, clamp = p.clamp_min == p.clamp_min;
#define VIG_WAVE2(TT, SO_)                                                             \
    if (raw) return clamp ? launch_wave<TT, true, true, SO_>(p, maps, ws, stream) : launch_wave<TT, true, false, SO_>(p, maps, ws, stream); \
    return clamp ? launch_wave<TT, false, true, SO_>(p, maps, ws, stream) : launch_wave<TT, false, false, SO_>(p, maps, ws, stream);
#define VIG_WAVE(TT) if (so) { VIG_WAVE2(TT, true) } VIG_WAVE2(TT, false)
    if (p.dtype == VIG_DTYPE_BF16) { VIG_WAVE(__nv_bfloat16) }
    VIG_WAVE(__half)
#undef VIG_WAVE
#undef VIG_WAVE2
}

}  // namespace vig

