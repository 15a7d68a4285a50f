// Bi-directional gated linear attention, warp-specialised "wavefront" form for large batches (tcgen05 + TMEM).
//
// Work item = (sequence b*h, segment of 256 tokens, direction).  Items are drawn from a ticket counter in
// wavefront order: step w holds segment w of every forward chain and segment nseg-1-w of every backward chain, so
// the state that enters an item was produced by an item with a smaller ticket, which is running or done.  States
// pass from segment to segment through a two-slot mailbox per (sequence, direction) in global memory; the two
// directions of a chunk meet in the output tensor: the direction that is scheduled first stores its half, the other
// adds to it with a vector reduction once the first has raised the chunk's flag.
//
// One persistent CTA per SM runs a pipeline over its stream of chunk iterations, roles decoupled by mbarriers:
//
//   load thread       work tickets; TMA loads of q, k, gates, v into a 3-stage ring
//   MMA thread        all tcgen05.mma issue (both threads sit in a fifth warpgroup that is otherwise idle)
//   8 prep warps      cumulative log-gates, q * 2^(G_i - G_ref) and k * 2^(G_ref - G_j) IN PLACE over the raw tiles
//   4 score warps     scores TMEM -> masked bf16 tiles; output accumulators TMEM -> global (store or reduction)
//   4 state warps     S <- 2^G_last S + 2^(G_last - G_ref) K~^T V in registers; bf16 state operand; mailbox
//
// Per iteration m (one chunk of 128 tokens, one direction), on the tensor core:
//   P  = Q~ K~^T                (128x128x64)   then masked by the score warps
//   O  = Q~ (2^G_ref S_in)      (128x 64x64)   skipped when S_in is exactly zero
//   O += P V                    (128x 64x128)
//   U  = K~^T V                 ( 64x 64x128)
// Only the state chain (U -> S -> state operand -> next chunk's second product) is sequential; everything else of
// the following iterations runs ahead as far as the rings allow.
//
// Every wait (mbarrier, mailbox counter, chunk flag) is bounded; when one runs out the CTA sets bit 0 of the status
// word, stops waiting on anything else, drains its control flow and frees its tensor memory.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int WDK = 64, WDV = 64;
constexpr int W_SEG_CHUNKS = 2, W_SEG = CHUNK * W_SEG_CHUNKS;
constexpr int W_PREP_WARPS = 8, W_THREADS = 20 * 32;      // five warpgroups: prep, prep, score, state, control
constexpr int W_STAGES = 3;
// Registers per thread.  The kernel is compiled and launched with W_REGS_BASE for all five warpgroups (five warps
// per scheduler allow no more); the control warpgroup gives most of its share back and the prep and score warpgroups
// take it.  An increase waits until the registers are there, so the shares must never add up to more than was
// launched with.
constexpr int W_REGS_BASE = 96, W_REGS_PREP = 112, W_REGS_SCORE = 120, W_REGS_STATE = W_REGS_BASE, W_REGS_CTRL = 40;
static_assert(2 * W_REGS_PREP + W_REGS_SCORE + W_REGS_STATE + W_REGS_CTRL <= 5 * W_REGS_BASE, "register shares exceed the launch allocation");
constexpr int W_TILE = CHUNK * 128;                           // 16 KB: 128 rows x 128 B
constexpr int W_STAGE_B = 4 * W_TILE;                         // q | k | gates | v
constexpr int WS_Q = 0, WS_K = W_TILE, WS_G = 2 * W_TILE, WS_V = 3 * W_TILE;
constexpr int WO_X = W_STAGES * W_STAGE_B;                    // score tile of key columns 64..127 (0..63 go over the dead gate tile)
constexpr int WO_ST = WO_X + W_TILE;                          // bf16 state operand, 64 rows x 128 B
constexpr int WO_PART = WO_ST + 64 * 128;                     // fp32 [2][8][64] group sums of log-gates
constexpr int WO_VEC = WO_PART + 2 * 8 * 64 * 4;              // fp32 [4][4][64]: 2^G_last, 2^(G_last-G_ref), G_ref, G_last per iteration
constexpr int WO_ITEMS = WO_VEC + 4 * 4 * 64 * 4;             // ring of 8 work items x 8 ints
constexpr int WO_BAR = WO_ITEMS + 8 * 32;
constexpr int WO_MISC = WO_BAR + 32 * 8;                      // tmem base, abort flag
constexpr int W_SMEM_BYTES = WO_MISC + 16 + 1024;             // + slack for the manual 1024-byte alignment

// TMEM columns (fp32): scores, state update, two output slots
constexpr uint32_t WT_P = 0, WT_U = 128, WT_O = 192, WT_COLS = 512;

// mbarrier indices
enum { B_FULL = 0, B_SFREE = 3, B_PREPPED = 6, B_PFULL = 9, B_PREADY = 10, B_STREADY = 11, B_UFULL = 12, B_OFULL = 13, B_OFREE = 15, B_PART = 17, B_COUNT = 18 };

struct WaveParams {
    BiglaParams p;
    uint32_t* ticket;      // [1]
    uint32_t* chain_cnt;   // [B*H][2]: state warps that have published step w (4 per step)
    uint32_t* chunk_flag;  // [B*H][nseg*2]: score warps of the first direction that have stored the chunk (4 = done)
    float* mailbox;        // [B*H][2 dirs][2 slots][dk*dv + dk]
    int nseg;
};

struct Item { int bh, seg, dir, nch, w, pad0, pad1, pad2; };


template <typename T> struct RedAdd;
template <> struct RedAdd<__nv_bfloat16> {
    __device__ static void v4(void* p, uint4 w) {
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
    }
};
template <> struct RedAdd<__half> {
    __device__ static void v4(void* p, uint4 w) {
        asm volatile("red.relaxed.gpu.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
    }
};

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


template <typename T>
__global__ void __launch_bounds__(W_THREADS, 1) bigla_wave_kernel(const __grid_constant__ TcMaps maps, const WaveParams wp) {
    const BiglaParams& p = wp.p;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nseg = wp.nseg;
    const int dir_first = (p.dir_mask & 1) ? 0 : 1, ndir = (p.dir_mask == 3) ? 2 : 1;
    const int per_step = p.B * p.H * ndir, total = per_step * nseg;

    auto bar = [&](int i) { return sbase + WO_BAR + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + WO_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + WO_MISC + 4);
    volatile Item* ring = reinterpret_cast<volatile Item*>(smem + WO_ITEMS);
    float* vec = reinterpret_cast<float*>(smem + WO_VEC);
    const Waiter waiter{abort_flag, p.status};

    if (tid == 0) {
        for (int i = 0; i < 3; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_SFREE + i), 1); mbar_init(bar(B_PREPPED + i), W_PREP_WARPS); }
        mbar_init(bar(B_PART), W_PREP_WARPS);
        mbar_init(bar(B_PFULL), 1); mbar_init(bar(B_PREADY), 4); mbar_init(bar(B_STREADY), 4); mbar_init(bar(B_UFULL), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_OFULL + i), 1); mbar_init(bar(B_OFREE + i), 4); }
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
        it.bh = r->bh; it.seg = r->seg; it.dir = r->dir; it.nch = r->nch; it.w = r->w;
    };
    // chunk (inside its segment) of sweep position ci, and its first token
    auto chunk_of = [&](const Item& it, int ci) { return it.dir ? it.nch - 1 - ci : ci; };
    auto state_zero = [&](const Item& it, int ci) { return ci == 0 && it.w == 0 && (it.dir ? p.init_b : p.init_f) == nullptr; };

    constexpr uint32_t IDESC_QK = make_idesc(Pack2<T>::FMT, 0, 0, 128, 128);
    constexpr uint32_t IDESC_OV = make_idesc(Pack2<T>::FMT, 0, 1, 128, 64);
    constexpr uint32_t IDESC_U = make_idesc(Pack2<T>::FMT, 1, 1, 64, 64);

    if (warp >= 16) {
        // =============================== control warpgroup ===============================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(W_REGS_CTRL));
        if (tid == 17 * 32) {
            // ---- load thread: work tickets and TMA loads, up to W_STAGES iterations ahead of the tensor core ----
            int tk = (int)atomicAdd(wp.ticket, 1u);
            int tk_next = (int)atomicAdd(wp.ticket, 1u);       // consumed one item later: its round trip costs no stall
            Item lcur; lcur.nch = 0; lcur.bh = lcur.seg = lcur.dir = lcur.w = 0;
            int l_items = 0, l_ci = 0;
            #pragma unroll 1
            for (uint32_t lm = 0;; ++lm, ++l_ci) {
                if (l_ci == lcur.nch) {                        // next work item
                    const int t = tk;
                    tk = tk_next;
                    tk_next = (int)atomicAdd(wp.ticket, 1u);
                    if (t < total) {
                        lcur.w = t / per_step;
                        const int r = t % per_step;
                        lcur.bh = r / ndir;
                        lcur.dir = dir_first + r % ndir;
                        lcur.seg = lcur.dir ? nseg - 1 - lcur.w : lcur.w;
                        lcur.nch = min(W_SEG_CHUNKS, (p.L - lcur.seg * W_SEG + CHUNK - 1) / CHUNK);
                    } else {
                        lcur.nch = 0;
                    }
                    volatile Item* r = ring + (l_items & 7);
                    r->bh = lcur.bh; r->seg = lcur.seg; r->dir = lcur.dir; r->nch = lcur.nch; r->w = lcur.w;
                    ++l_items;
                    l_ci = 0;
                }
                const uint32_t s = lm % 3;
                if (lm >= 3) waiter.wait_lite(bar(B_SFREE + s), ((lm / 3) - 1) & 1);
                if (*abort_flag) break;
                if (lcur.nch == 0) { mbar_arrive_plain(bar(B_FULL + s)); break; }   // end marker: wakes the prep warps
                const int t0 = lcur.seg * W_SEG + chunk_of(lcur, l_ci) * CHUNK;
                const int b = lcur.bh / p.H, h = lcur.bh % p.H;
                const uint32_t dst = sbase + s * W_STAGE_B, fb = bar(B_FULL + s);
                mbar_expect_tx(fb, W_STAGE_B);
                tma_load_4d(dst + WS_K, &maps.k, 0, t0, h, b, fb);
                tma_load_4d(dst + WS_G, lcur.dir ? &maps.gb : &maps.gf, 0, t0, h, b, fb);
                tma_load_4d(dst + WS_Q, &maps.q, 0, t0, h, b, fb);
                tma_load_4d(dst + WS_V, &maps.v, 0, t0, h, b, fb);
            }
        } else if (tid == 16 * 32) {
            // ---- MMA thread ----
            Item mcur; mcur.nch = 0; mcur.bh = mcur.seg = mcur.dir = mcur.w = 0;
            int m_items = 0, m_ci = 0;
            #pragma unroll 1
            for (uint32_t m = 0;; ++m, ++m_ci) {
                const uint32_t s = m % 3, st = sbase + s * W_STAGE_B;
                waiter.wait_lite(bar(B_PREPPED + s), (m / 3) & 1);  // also orders the read of the work item after its write
                if (*abort_flag) break;
                if (m_ci == mcur.nch) { read_item(m_items, mcur); ++m_items; m_ci = 0; }
                if (mcur.nch == 0) { mbar_arrive_plain(bar(B_PFULL)); break; }      // end marker: wakes the score warps
                const uint32_t qt = st + WS_Q, kt = st + WS_K, vt = st + WS_V, p0 = st + WS_G, p1 = sbase + WO_X, stt = sbase + WO_ST;
                const uint32_t o_acc = tmem + WT_O + 64u * (m & 1u);
                const bool s_zero = state_zero(mcur, m_ci);
                // (a) scores
                tc_fence_after();
#pragma unroll 1
                for (int k4 = 0; k4 < WDK / 16; ++k4) tc_mma(tmem + WT_P, make_desc(qt + k4 * 32), make_desc(kt + k4 * 32), IDESC_QK, k4 > 0);
                tc_commit(bar(B_PFULL));
                // (b) product with the entering state
                waiter.wait_lite(bar(B_STREADY), m & 1);
                if (m >= 2) waiter.wait_lite(bar(B_OFREE + (m & 1)), ((m >> 1) - 1) & 1);
                tc_fence_after();
                if (!s_zero) {
#pragma unroll 1
                    for (int k4 = 0; k4 < WDK / 16; ++k4) tc_mma(o_acc, make_desc(qt + k4 * 32), make_desc(stt + k4 * 2048), IDESC_OV, k4 > 0);
                }
                // (c) masked scores x v, state update
                waiter.wait_lite(bar(B_PREADY), m & 1);
                tc_fence_after();
#pragma unroll 1
                for (int k8 = 0; k8 < CHUNK / 16; ++k8)
                    tc_mma(o_acc, make_desc((k8 < 4 ? p0 : p1) + (k8 & 3) * 32), make_desc(vt + k8 * 2048), IDESC_OV, !s_zero || k8 > 0);
                tc_commit(bar(B_OFULL + (m & 1)));
#pragma unroll 1
                for (int k8 = 0; k8 < CHUNK / 16; ++k8)
                    tc_mma(tmem + WT_U, make_desc(kt + k8 * 2048), make_desc(vt + k8 * 2048), IDESC_U, k8 > 0);
                tc_commit(bar(B_UFULL));
                tc_commit(bar(B_SFREE + s));
            }
        }
    } else if (warp < W_PREP_WARPS) {
        // =============================== prep warps: gates and operand scaling, in place ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(W_REGS_PREP));
        constexpr int NG = 8;                                 // groups (of 16 tokens, one per warp) per chunk
        const int grp = warp;
        const bool raw_logits = p.gate_norm > 0.f;
        const float inv_norm = raw_logits ? 1.f / p.gate_norm : 1.f;
        const float clamp_lo = (p.clamp_min == p.clamp_min) ? p.clamp_min * LOG2E : -INFINITY;
        Item cur; cur.nch = 0; cur.bh = cur.seg = cur.dir = cur.w = 0;
        int items = 0, ci = 0;
        #pragma unroll 1
        for (uint32_t m = 0;; ++m, ++ci) {
            const uint32_t s = m % 3;
            if (lane == 0) waiter.wait_lite(bar(B_FULL + s), (m / 3) & 1);
            __syncwarp();
            if (*abort_flag) break;
            if (ci == cur.nch) { read_item(items, cur); ++items; ci = 0; }
            if (cur.nch == 0) { if (lane == 0) mbar_arrive_plain(bar(B_PREPPED + s)); break; }
            uint8_t* stg = smem + s * W_STAGE_B;
            const uint32_t* sg = reinterpret_cast<const uint32_t*>(stg + WS_G);
            float* part = reinterpret_cast<float*>(smem + WO_PART) + (m & 1) * (NG * WDK);
            const int t0 = cur.seg * W_SEG + chunk_of(cur, ci) * CHUNK;
            const int n_valid = p.L - t0;                     // rows at or past it are padding: decay 1
            // ONE code path for both directions and for clamped / padded chunks (runtime selects instead of template
            // variants): the five roles of this CTA run different code at the same time, and what does not fit the
            // instruction cache stalls all of them.
            // A warp owns 16 tokens (one group); a half-warp covers one token row with 4 channels per lane (8-byte
            // accesses), so a lane handles 8 consecutive scan positions x 4 channels and the per-token overhead
            // (addresses, padding test) is paid once per 4 channels.  Scan position sp = 8*half + u is token
            // 16*warp + (sp ^ dmask).
            const int dir = cur.dir;
            const int dmask = dir ? 15 : 0;
            const int half = lane >> 4, c4l = lane & 15;      // my half of the group, my 4 channels: 4*c4l .. 4*c4l+3
            const uint32_t sw_chunk = (uint32_t)c4l >> 1, sw_in = (uint32_t)(c4l & 1) * 8;
            float4 half_off;                                  // sum of the other half-warp's tokens when they precede mine in the scan
            // The 8 tokens of a lane are handled as two halves of 4 by loops that run twice; the cumulative gates of the
            // halves rotate through two register arrays (glA = first half, glB = second), so the loop bodies are half the
            // code of a full unroll while four tokens x four channels still overlap their latencies.
            float4 glA[4], glB[4];
            {
                float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) glA[i] = glB[i];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int tok = warp * 16 + ((half * 8 + hh * 4 + i) ^ dmask);
                        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(sg) + tok * 128 + c4l * 8);
                        const float2 a = Pack2<T>::unpack(raw.x), b2 = Pack2<T>::unpack(raw.y);
                        float4 g;
                        g.x = fmaxf(gate2_short(a.x, raw_logits, -inv_norm), clamp_lo);
                        g.y = fmaxf(gate2_short(a.y, raw_logits, -inv_norm), clamp_lo);
                        g.z = fmaxf(gate2_short(b2.x, raw_logits, -inv_norm), clamp_lo);
                        g.w = fmaxf(gate2_short(b2.y, raw_logits, -inv_norm), clamp_lo);
                        if (tok >= n_valid) g = make_float4(0.f, 0.f, 0.f, 0.f);
                        run.x += g.x; run.y += g.y; run.z += g.z; run.w += g.w;
                        glB[i] = run;
                    }
                }
                // the second half-warp continues the first half-warp's sum; it also knows the group's total
                float4 first;
                first.x = __shfl_sync(0xffffffffu, run.x, c4l); first.y = __shfl_sync(0xffffffffu, run.y, c4l);
                first.z = __shfl_sync(0xffffffffu, run.z, c4l); first.w = __shfl_sync(0xffffffffu, run.w, c4l);
                if (half) reinterpret_cast<float4*>(part)[grp * 16 + c4l] = make_float4(run.x + first.x, run.y + first.y, run.z + first.z, run.w + first.w);
                if (!half) first = make_float4(0.f, 0.f, 0.f, 0.f);
                half_off = first;                             // joins the group offset below
            }
            // the prep warps meet on an mbarrier, not a named barrier: its wait is bounded like every other wait here
            __syncwarp();
            if (lane == 0) { mbar_arrive_plain(bar(B_PART)); waiter.wait_lite(bar(B_PART), m & 1); }
            __syncwarp();
            float4 off = half_off, gref = make_float4(0.f, 0.f, 0.f, 0.f), glast = gref;
#pragma unroll 2
            for (int g2 = 0; g2 < NG; ++g2) {
                const float4 s4 = reinterpret_cast<const float4*>(part)[g2 * 16 + c4l];
                const bool before = dir ? g2 > grp : g2 < grp;            // scanned before my group
                const bool in_ref = dir ? g2 >= NG / 2 : g2 < NG / 2;     // part of the cumulative gate at the middle token
                if (before) { off.x += s4.x; off.y += s4.y; off.z += s4.z; off.w += s4.w; }
                if (in_ref) { gref.x += s4.x; gref.y += s4.y; gref.z += s4.z; gref.w += s4.w; }
                glast.x += s4.x; glast.y += s4.y; glast.z += s4.z; glast.w += s4.w;
            }
            off.x -= gref.x; off.y -= gref.y; off.z -= gref.z; off.w -= gref.w;
            // Log-gates are <= 0, so a lane's exponents are monotone along its 8 tokens: the largest magnitude (for the
            // status flag; every exponent is clamped regardless) is at one of the two ends.
            float worst = fmaxf(fmaxf(fabsf(off.x + glA[0].x), fabsf(off.y + glA[0].y)), fmaxf(fabsf(off.z + glA[0].z), fabsf(off.w + glA[0].w)));
            worst = fmaxf(worst, fmaxf(fmaxf(fabsf(off.x + glB[3].x), fabsf(off.y + glB[3].y)), fmaxf(fabsf(off.z + glB[3].z), fabsf(off.w + glB[3].w))));
            auto clampx = [](float e) { return fminf(fmaxf(e, -MAX_EXPONENT2), MAX_EXPONENT2); };
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {
                uint2 rk[4], rq[4];
                uint32_t offs[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {                 // all reads before the writes: the tiles alias for the compiler
                    const uint32_t tok = (uint32_t)(warp * 16 + ((half * 8 + hh * 4 + i) ^ dmask));
                    offs[i] = tok * 128 + ((sw_chunk ^ (tok & 7)) << 4) + sw_in;
                    rk[i] = *reinterpret_cast<const uint2*>(stg + WS_K + offs[i]);
                    rq[i] = *reinterpret_cast<const uint2*>(stg + WS_Q + offs[i]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float ex = clampx(off.x + glA[i].x), ey = clampx(off.y + glA[i].y), ez = clampx(off.z + glA[i].z), ew = clampx(off.w + glA[i].w);
                    // fp32 products, one rounding to the 16-bit operand; scale * out_scale is applied to the output instead
                    const float2 k0 = Pack2<T>::unpack(rk[i].x), k1 = Pack2<T>::unpack(rk[i].y);
                    const float2 q0 = Pack2<T>::unpack(rq[i].x), q1 = Pack2<T>::unpack(rq[i].y);
                    uint2 ko, qo;
                    ko.x = Pack2<T>::pack(k0.x * ex2(-ex), k0.y * ex2(-ey)); ko.y = Pack2<T>::pack(k1.x * ex2(-ez), k1.y * ex2(-ew));
                    qo.x = Pack2<T>::pack(q0.x * ex2(ex), q0.y * ex2(ey)); qo.y = Pack2<T>::pack(q1.x * ex2(ez), q1.y * ex2(ew));
                    *reinterpret_cast<uint2*>(stg + WS_K + offs[i]) = ko;
                    *reinterpret_cast<uint2*>(stg + WS_Q + offs[i]) = qo;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) glA[i] = glB[i];
            }
            if (grp == 0 && half == 0) {                      // per-channel factors of this iteration for the state warps
                float* ve = vec + (m & 3) * 256 + 4 * c4l;
                *reinterpret_cast<float4*>(ve) = make_float4(ex2(glast.x), ex2(glast.y), ex2(glast.z), ex2(glast.w));
                *reinterpret_cast<float4*>(ve + 64) = make_float4(ex2(glast.x - gref.x), ex2(glast.y - gref.y), ex2(glast.z - gref.z), ex2(glast.w - gref.w));
                *reinterpret_cast<float4*>(ve + 128) = gref;
                *reinterpret_cast<float4*>(ve + 192) = glast;
            }
            const bool out_of_range = worst > MAX_EXPONENT2;
            if (out_of_range && p.status) atomicOr(p.status, 2);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar(B_PREPPED + s));
        }
    } else if (warp < W_PREP_WARPS + 4) {
        // =============================== score warps: masking, output ===============================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(W_REGS_SCORE));
        const int quad = warp & 3;                            // my 32 query rows and TMEM lanes
        const int row = 32 * quad + lane;
        const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
        const float o_sign = p.qscale;                        // scale * out_scale, applied to the finished accumulators
        Item cur; cur.nch = 0; cur.bh = cur.seg = cur.dir = cur.w = 0;
        Item prev = cur;
        int items = 0, ci = 0, prev_ci = 0;
        // output of iteration j: accumulator slot j & 1 -> global
        auto epilogue = [&](uint32_t j, const Item& it, int jci) {
            if (lane == 0) waiter.wait_lite(bar(B_OFULL + (j & 1)), (j >> 1) & 1);
            __syncwarp();
            tc_fence_after();
            const int c = chunk_of(it, jci);
            const int tok = it.seg * W_SEG + c * CHUNK + row;
            const int w_other = nseg - 1 - it.w;
            const bool first = ndir == 1 || it.w < w_other || (it.w == w_other && it.dir == 0);
            uint32_t* flag = wp.chunk_flag + (size_t)it.bh * nseg * W_SEG_CHUNKS + it.seg * W_SEG_CHUNKS + c;
            if (!first) {                                     // the other direction's half must be in place
                if (lane == 0) global_wait(flag, 4u, abort_flag);
                __syncwarp();
            }
            T* obase = reinterpret_cast<T*>(p.o) + (it.bh / p.H) * p.so[0] + (it.bh % p.H) * p.so[1] + (int64_t)tok * p.so[2];
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                float a[32];
                tc_ld32(tmem + lane_base + WT_O + 64u * (j & 1u) + 32 * half, a);
                tc_wait_ld();
                if (half == 1) {                              // the slot is read: hand it back before the global traffic
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_plain(bar(B_OFREE + (j & 1)));
                }
                if (tok < p.L) {
#pragma unroll
                    for (int q4 = 0; q4 < 32; q4 += 8) {
                        uint4 w4;
                        w4.x = Pack2<T>::pack(o_sign * a[q4], o_sign * a[q4 + 1]); w4.y = Pack2<T>::pack(o_sign * a[q4 + 2], o_sign * a[q4 + 3]);
                        w4.z = Pack2<T>::pack(o_sign * a[q4 + 4], o_sign * a[q4 + 5]); w4.w = Pack2<T>::pack(o_sign * a[q4 + 6], o_sign * a[q4 + 7]);
                        T* dst = obase + 32 * half + q4;
                        if (first) *reinterpret_cast<uint4*>(dst) = w4; else RedAdd<T>::v4(dst, w4);
                    }
                }
            }
            if (first && ndir == 2) {                         // publish my half of the chunk
                __syncwarp();
                if (lane == 0) { __threadfence(); atomicAdd(flag, 1u); }
            }
        };
        #pragma unroll 1
        for (uint32_t m = 0;; ++m, ++ci) {
            if (lane == 0) waiter.wait_lite(bar(B_PFULL), m & 1);
            __syncwarp();
            if (*abort_flag) break;
            if (ci == cur.nch) { read_item(items, cur); ++items; ci = 0; }
            const bool at_end = cur.nch == 0;
            if (!at_end) {
            tc_fence_after();
            uint8_t* p0 = smem + (m % 3) * W_STAGE_B + WS_G;  // keys 0..63 over the dead gate tile
            uint8_t* p1 = smem + WO_X;                        // keys 64..127
            // A 32x32 block of scores is wholly kept, wholly masked, or on the diagonal (warp-uniform test); on the
            // diagonal, bit j of `dmask_bits` says whether key j of the block is kept for my query row.
            const int dir = cur.dir;
            const uint32_t dmask_bits = dir ? ~((1u << lane) - 1u) : (lane == 31 ? 0xffffffffu : (2u << lane) - 1u);
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {                  // key block: keys 32*cb .. 32*cb+31
                if (cb == 2 && m > 0) {                       // the second tile is free once the previous iteration's MMAs are done
                    if (lane == 0) waiter.wait_lite(bar(B_UFULL), (m - 1) & 1);
                    __syncwarp();
                }
                const bool all_zero = dir ? cb < quad : cb > quad;
                uint8_t* prow = (cb < 2 ? p0 : p1) + row * 128;
                const uint32_t chunk0 = (uint32_t)(cb & 1) * 4;           // first 16-byte chunk of this block in the 128-byte row
                if (all_zero) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(prow + (((chunk0 + j) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                } else {
                    float a[32];
                    tc_ld32(tmem + lane_base + WT_P + 32 * cb, a);
                    tc_wait_ld();
                    if (cb == quad) {                                     // the diagonal block: per-element mask
#pragma unroll
                        for (int e = 0; e < 32; ++e) a[e] = (dmask_bits >> e) & 1u ? a[e] : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 w4;
                        w4.x = Pack2<T>::pack(a[8 * j], a[8 * j + 1]); w4.y = Pack2<T>::pack(a[8 * j + 2], a[8 * j + 3]);
                        w4.z = Pack2<T>::pack(a[8 * j + 4], a[8 * j + 5]); w4.w = Pack2<T>::pack(a[8 * j + 6], a[8 * j + 7]);
                        *reinterpret_cast<uint4*>(prow + (((chunk0 + j) ^ (row & 7)) << 4)) = w4;
                    }
                }
            }
            tc_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar(B_PREADY));
            }
            if (m > 0) epilogue(m - 1, prev, prev_ci);       // one iteration behind: the MMAs of m - 1 finish meanwhile
            if (at_end) break;
            prev = cur; prev_ci = ci;
        }
    } else if (warp < W_PREP_WARPS + 8) {
        // =============================== state warps ===============================
        const int quad = warp & 3;
        const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
        const int st_row = 16 * quad + (lane & 15);           // key channel: an M=64 accumulator puts row r in lane (r%16) + 32*(r/16)
        const int hi = lane >> 4;                             // lanes 16-31 take columns 16..31 and 48..63 of the same rows
        auto col_of = [&](int j) { return 32 * (j >> 4) + 16 * hi + (j & 15); };
        constexpr int NE = WDK * WDV, SLOT = NE + WDK;
        float S[32];
        float gacc = 0.f;                                     // summed log2-gates of my channel along the chain so far
        Item cur; cur.nch = 0; cur.bh = cur.seg = cur.dir = cur.w = 0;
        int items = 0, ci = 0;
        bool s_zero = true;
        #pragma unroll 1
        for (uint32_t m = 0;; ++m, ++ci) {
            const uint32_t s = m % 3;
            if (lane == 0) waiter.wait_lite(bar(B_PREPPED + s), (m / 3) & 1);
            __syncwarp();
            if (*abort_flag) break;
            if (ci == cur.nch) { read_item(items, cur); ++items; ci = 0; }
            if (cur.nch == 0) break;
            if (ci == 0) {                                    // the chain enters a new segment
                const float* src = nullptr;
                if (cur.w == 0) {
                    const float* init = cur.dir ? p.init_b : p.init_f;
                    if (init) src = init + (size_t)cur.bh * NE;
                    gacc = 0.f;
                } else {
                    uint32_t* cnt = wp.chain_cnt + cur.bh * 2 + cur.dir;
                    if (lane == 0) global_wait(cnt, 4u * (uint32_t)cur.w, abort_flag);
                    __syncwarp();
                    const float* box = wp.mailbox + (((size_t)cur.bh * 2 + cur.dir) * 2 + ((cur.w - 1) & 1)) * SLOT;
                    src = box;
                    gacc = __ldcg(box + NE + st_row);
                }
                s_zero = src == nullptr;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 t4 = src ? __ldcg(reinterpret_cast<const float4*>(src + st_row * WDV + col_of(j))) : make_float4(0.f, 0.f, 0.f, 0.f);
                    S[j] = t4.x; S[j + 1] = t4.y; S[j + 2] = t4.z; S[j + 3] = t4.w;
                }
            }
            const float* ve = vec + (m & 3) * 256;
            if (!s_zero) {                                    // bf16(2^G_ref * S_in), MN-major [channel][value]
                const float eg = ex2(ve[128 + st_row]);
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
            if (lane == 0) waiter.wait_lite(bar(B_UFULL), m & 1);
            __syncwarp();
            tc_fence_after();
            {
                const float e_last = ve[st_row], e_rel = ve[64 + st_row];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    float u[32];
                    tc_ld32(tmem + lane_base + WT_U + 32 * half, u);   // rows live in lanes 0-15 of the warp
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float up = __shfl_sync(0xffffffffu, u[16 + j], lane & 15);   // columns 16-31 go to lanes 16-31
                        const float mine = hi ? up : u[j];
                        S[16 * half + j] = fmaf(S[16 * half + j], e_last, e_rel * mine);
                    }
                }
                gacc += ve[192 + st_row];
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
                    if (fin) dst = fin + (size_t)cur.bh * NE;
                    if (ld) gdst = ld + (size_t)cur.bh * WDK;
                } else {
                    float* box = wp.mailbox + (((size_t)cur.bh * 2 + cur.dir) * 2 + (cur.w & 1)) * SLOT;
                    dst = box; gdst = box + NE;
                }
                if (dst) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(dst + st_row * WDV + col_of(j)) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
                }
                if (gdst && hi == 0) gdst[st_row] = last ? gacc * LN2 : gacc;   // the caller gets natural-log units
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

size_t wave_counter_bytes(int B, int H, int nseg) {
    return ((1 + 2 * (size_t)B * H + (size_t)B * H * nseg * W_SEG_CHUNKS) * sizeof(uint32_t) + 255) & ~(size_t)255;
}

template <typename T>
int launch_wave(const BiglaParams& p, const TcMaps& maps, void* ws, cudaStream_t stream) {
    const int nseg = (p.L + W_SEG - 1) / W_SEG;
    const int BH = p.B * p.H;
    WaveParams wp;
    wp.p = p;
    wp.nseg = nseg;
    wp.ticket = reinterpret_cast<uint32_t*>(ws);
    wp.chain_cnt = wp.ticket + 1;
    wp.chunk_flag = wp.chain_cnt + 2 * (size_t)BH;
    const size_t cb = wave_counter_bytes(p.B, p.H, nseg);
    wp.mailbox = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + cb);
    cudaError_t e;
    if ((e = cudaMemsetAsync(ws, 0, cb, stream)) != cudaSuccess) return (int)e;
    static int sm_count[64] = {};
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return VIG_ERR_DEVICE;
    auto kern = bigla_wave_kernel<T>;
    if (!sm_count[dev]) {
        int sms = 0;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        sm_count[dev] = sms;
    }
    if ((e = ensure_smem_attr(reinterpret_cast<const void*>(kern), W_SMEM_BYTES)) != cudaSuccess) return (int)e;
    const int ndir = p.dir_mask == 3 ? 2 : 1;
    const long long items = (long long)BH * ndir * nseg;
    const int grid = (int)(items < sm_count[dev] ? items : sm_count[dev]);
    kern<<<grid, W_THREADS, W_SMEM_BYTES, stream>>>(maps, wp);
    return (int)cudaGetLastError();
}

}  // namespace

bool bigla_wave_supported(const BiglaParams& p) {
    if (p.dtype != VIG_DTYPE_BF16 && p.dtype != VIG_DTYPE_F16) return false;
    if (p.dv != WDV || p.dk != WDK || !p.o || !p.q || p.B * p.H < 1 || p.L < 1) return false;
    if (p.dir_mask < 1 || p.dir_mask > 3) return false;
    if (!tc::tma_ok(p.q, p.sq, p.B, p.H) || !tc::tma_ok(p.k, p.sk, p.B, p.H) || !tc::tma_ok(p.v, p.sv, p.B, p.H)) return false;
    if ((p.dir_mask & 1) && (!p.gf || !tc::tma_ok(p.gf, p.sgf, p.B, p.H))) return false;
    if ((p.dir_mask & 2) && (!p.gb || !tc::tma_ok(p.gb, p.sgb, p.B, p.H))) return false;
    if ((reinterpret_cast<uintptr_t>(p.o) & 15) || (p.so[0] * 2) % 16 || (p.so[1] * 2) % 16 || (p.so[2] * 2) % 16) return false;
    return tc::encode_fn() != nullptr;
}

// Measured on B200: with at least as many (sequence, direction) chains as SMs and two or more segments per sequence the
// wavefront form beats the segment-parallel forms (0.46 against 0.58 ms at 64 x 3 sequences of 4096 tokens); with
// fewer chains its CTAs idle, and a single segment has nothing to hand on.
bool bigla_wave_preferred(const BiglaParams& p) {
    static int sm_count[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!sm_count[dev]) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
        sm_count[dev] = sms;
    }
    const int ndir = p.dir_mask == 3 ? 2 : 1;
    return p.L > W_SEG && (long long)p.B * p.H * ndir >= sm_count[dev];
}

// Counters (ticket, chain progress, chunk flags) followed by the state mailboxes.
size_t bigla_wave_workspace(int B, int H, int L, int dk, int dv) {
    const int nseg = (L + W_SEG - 1) / W_SEG;
    return wave_counter_bytes(B, H, nseg) + (size_t)B * H * 2 * 2 * ((size_t)dk * dv + dk) * sizeof(float);
}

int bigla_wave_launch(const BiglaParams& p, void* ws, size_t ws_bytes, cudaStream_t stream) {
    if (!ws || ws_bytes < bigla_wave_workspace(p.B, p.H, p.L, p.dk, p.dv)) return VIG_ERR_WORKSPACE;
    tc::TcMaps maps;
    const void* gfs = p.gf ? p.gf : p.gb;
    const int64_t* gfst = p.gf ? p.sgf : p.sgb;
    const void* gbs = p.gb ? p.gb : p.gf;
    const int64_t* gbst = p.gb ? p.sgb : p.sgf;
    if (!tc::make_map(&maps.q, p.q, p.sq, p.B, p.H, p.L, p.dk, p.dtype, true) ||
        !tc::make_map(&maps.k, p.k, p.sk, p.B, p.H, p.L, p.dk, p.dtype, true) ||
        !tc::make_map(&maps.v, p.v, p.sv, p.B, p.H, p.L, p.dv, p.dtype, true) ||
        !tc::make_map(&maps.gf, gfs, gfst, p.B, p.H, p.L, p.dk, p.dtype, false) ||
        !tc::make_map(&maps.gb, gbs, gbst, p.B, p.H, p.L, p.dk, p.dtype, false))
        return VIG_ERR_DEVICE;
    if (p.dtype == VIG_DTYPE_BF16) return launch_wave<__nv_bfloat16>(p, maps, ws, stream);
    return launch_wave<__half>(p, maps, ws, stream);
}

}  // namespace vig

