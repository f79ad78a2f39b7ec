// Sparse convolution as an implicit GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces, for fp16 features and 16/32/64 channels, the reference's per-offset scalar kernel
// (submConv3dlayer.cu:479-518, launched kvol times per layer, :632-638). One CTA owns a tile of 128
// output rows. For every group of kernel offsets it gathers the 128 neighbour rows into shared
// memory as a K-major, 128-byte-swizzled A operand (one 128-byte row per output row: 64/Cin offsets
// side by side, missing neighbours zero-filled), streams the matching pre-tiled weight block as the B
// operand with a bulk asynchronous copy, and issues tcgen05.mma (M=128, N=Cout, K=16 x 4) into one
// fp32 accumulator in tensor memory that stays resident across all offsets. A CTA iteration covers
// four such tiles (512 rows, four accumulators) with the offset loop outermost, so that a weight block
// is fetched once per four tiles; (tile, offset group) pairs without any neighbour are skipped using
// the per-tile offset masks the rulebook kernels produce. The epilogue reads the
// accumulator with tcgen05.ld, applies the folded BatchNorm scale/shift and ReLU, and stores fp16
// rows (and, for the last layer, scatters them into the dense BEV map).
//
// Warp roles (256 threads, two CTAs per SM, about 85 KB of shared memory and at most 104 registers per
// thread, which leaves room for other streams' kernels on the same SM):
//   warps 0-3  gather. The ring has one 16 KB slot per gather warp; ring position q lives in slot q % 4
//              and is filled by warp q % 4 alone with 32 sixteen-byte cp.async per lane group. A warp's
//              cp.async issue rate is bound by latency (about 46 cycles per instruction), so the warps
//              work on four different stages at once rather than sharing one; the copies publish the
//              stage themselves (cp.async mbarrier arrival). After the group's last stage the four warps
//              run the epilogue (each can read its quarter of the tensor-memory lanes).
//   warps 4, 7 issue the MMAs of the even / odd row tiles from one thread each (one issue costs the
//              thread about 76 cycles, a commit about 156). Each issuer has its own "landed" barrier
//              per slot: a parity wait is only safe for a waiter that has seen every earlier phase.
//   warp 5     streams the weight blocks (cp.async.bulk), warp 6 prefetches the neighbour indices of
//              upcoming stages into a small shared-memory ring.
// A CTA walks an equal share of all occupied row tiles (row counts are read on the device). Every wait is
// bounded by a clock limit, after which the CTA raises SESSD_STATUS_TIMEOUT (and reports which wait in
// the status block), stops issuing work, frees its tensor memory and returns.
#include <atomic>
#include <cstdlib>
#include <string>
#include <vector>

#include "common.cuh"

namespace sessd {

namespace {

constexpr int TILE_M = 128;
constexpr int MMA_WARPS_MAX = 2;
constexpr int TILES = 4;                     // row tiles per CTA iteration; they share each weight block
constexpr int GATHER_WARPS = 4;               // warps 0-3: gather, later epilogue
constexpr int A_STAGES_MAX = GATHER_WARPS;
constexpr int B_STAGES = 2;
// One gather stage (16 KB) per gather warp: ring position q lives in slot q % 4 and is filled by warp q % 4, so
// every barrier of a slot has one producer warp that uses it in order. With the weight ring (2 x Cout x 128 B),
// the index ring and the control block a CTA takes about 85 KB of shared memory; two CTAs fit one SM.
constexpr int IDX_STAGES = 6;                // ring of neighbour-index blocks, filled ahead by the index warp
template <int CIN, int COUT>
struct RingCfg {
    static constexpr int A_STAGES = GATHER_WARPS;
};
constexpr int ROW_BYTES = 128;               // 64 halves per A/B row
constexpr int A_BYTES = TILE_M * ROW_BYTES;  // 16 KB
constexpr int UMMA_THREADS = 256;
constexpr int MMA_WARPS = 2;                 // MMA issuer warps (4 and 7); one takes the even row tiles, the other the odd ones
constexpr int KVOL_MAX = 27;
constexpr long long WAIT_LIMIT_CYCLES = 200000000LL;   // about a tenth of a second; real waits are microseconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Same, but the hardware may park the thread for up to `ns` nanoseconds while the phase is incomplete,
// so a waiting warp does not take issue slots from the warps that feed the pipeline.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the phase did not complete within the clock limit or the CTA is aborting.
// The polling loop is kept to a handful of instructions (abort flag and clock are looked at every 32
// polls): the role warps spend most of their life here and must not take the issue slots of the warps
// that feed the pipeline. RELAXED waits (roles with slack: weight and index prefetch) also sleep
// between polls.
template <bool RELAXED = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (RELAXED) __nanosleep(200);
            if (mbar_try_wait_parked(bar, parity, 1000u)) return true;
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            if (*abort_flag == 0) abort_flag[1] = where;   // abort_where follows abort_flag in SharedCtl
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// 16-byte copy that writes zeros instead when index < 0 (the source address is then not touched).
__device__ __forceinline__ void cp_async_16_or_zero(uint32_t dst, const void* src, int index) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.lt.s32 p, %2, 0;\n\t"
        "cp.async.cg.shared.global [%0], [%1], 16, p;\n\t}" ::"r"(dst),
        "l"(src), "r"(index)
        : "memory");
}
// Arrival on `bar` that fires when all cp.async copies this thread has issued so far have landed
// (the barrier's expected count must include it).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024
// bytes apart (stride byte offset), leading byte offset unused by swizzled K-major layouts (set to 1),
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: fp32 accumulate, fp16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct SharedCtl {
    // a_full[i][s]: stage s has landed, for MMA issuer i (the issuer that owns the stage's row tile). One
    // barrier per (issuer, slot) keeps a single consumer per barrier: parity waits are only safe when the
    // waiter has itself seen every earlier phase complete.
    unsigned long long a_full[MMA_WARPS_MAX][A_STAGES_MAX];
    unsigned long long a_empty[A_STAGES_MAX];
    unsigned long long b_full[B_STAGES];
    unsigned long long b_empty[B_STAGES];
    unsigned long long i_full[IDX_STAGES];
    unsigned long long i_empty[IDX_STAGES];
    unsigned long long acc_full;
    unsigned long long acc_empty;
    unsigned long long mma_drain;   // aborting CTA only: completes when the issuers' outstanding MMAs have finished
    uint32_t tmem_base;
    int abort_flag;
    int abort_where;   // code of the first wait that ran out (role and ring position), for the status block
    // per gather warp: the (stage << 2 | tile) pairs of the current group in ring order, so that a warp
    // steps straight to the stages it owns
    uint8_t stage_list[GATHER_WARPS][TILES * 32];
#ifdef SESSD_UMMA_TIMING
    long long t_issue[A_STAGES_MAX];    // when the gathers of the stage were issued
    long long t_commit[A_STAGES_MAX];   // when the MMAs reading the stage were committed
#endif
};

template <int CIN, int COUT>
constexpr int umma_smem_bytes() {
    return 1024 /*alignment slack*/ + RingCfg<CIN, COUT>::A_STAGES * A_BYTES + B_STAGES * COUT * ROW_BYTES +
           IDX_STAGES * (64 / CIN) * TILE_M * 4 + 2 * COUT * 4 + (int)sizeof(SharedCtl);
}

// Offsets g*KG .. g*KG+KG-1 of a tile's 27-bit offset mask.
template <int KG>
__device__ __forceinline__ bool stage_active(uint32_t kmask, int g) {
    return ((kmask >> (g * KG)) & ((1u << KG) - 1u)) != 0u;
}

// Bit t set when row tile t has a neighbour under the offsets of stage g. The masks are only ever indexed
// with compile-time constants, so they stay in registers (local memory would miss in the small L1 that
// is left beside 200 KB of shared memory).
template <int KG>
__device__ __forceinline__ uint32_t active_tiles(const uint32_t (&m)[TILES], int g) {
    uint32_t bits = 0;
#pragma unroll
    for (int t = 0; t < TILES; ++t) bits |= (stage_active<KG>(m[t], g) ? 1u : 0u) << t;
    return bits;
}

// Advances to the next (stage g, tile t) pair with work, in the order stage-major, tile-minor; `rem` holds
// the tiles of stage g not yet visited. Start with g = -1, rem = 0.
template <int KG>
__device__ __forceinline__ bool next_item(const uint32_t (&m)[TILES], int nstages, int& g, uint32_t& rem, int& t) {
    while (rem == 0u) {
        if (++g >= nstages) return false;
        rem = active_tiles<KG>(m, g);
    }
    t = __ffs((int)rem) - 1;
    rem &= rem - 1u;
    return true;
}

// Register cap well below what two resident CTAs (the shared-memory limit) could take: the rest of the
// register file is what lets blocks of other kernels (other streams) run beside them.
template <int CIN, int COUT>
__global__ void __maxnreg__(104)
conv_umma_kernel(const __half* __restrict__ in, __half* __restrict__ out, const int32_t* __restrict__ nbr,
                 const uint32_t* __restrict__ tile_mask, const int32_t* __restrict__ out_num,
                 const uint8_t* __restrict__ wtiles, const float* __restrict__ scale, const float* __restrict__ shift,
                 int relu, int batch, int max_voxels, int kvol, __half* __restrict__ dense,
                 const int4* __restrict__ out_coors, int D, int H, int W, int32_t* status, int withhold_weights) {
    // withhold_weights (tests of the time-out path only): the weight streamer stays silent, so the MMA issuers'
    // bounded wait for the first weight block runs out and every CTA with work leaves through the abort path.
    constexpr int KG = 64 / CIN;            // kernel offsets sharing one 128-byte A row
    constexpr int CPO = CIN / 8;            // 16-byte chunks per offset
    constexpr int B_BYTES = COUT * ROW_BYTES;
    constexpr int A_STAGES = RingCfg<CIN, COUT>::A_STAGES;
    constexpr int IDX_WORDS = KG * TILE_M;  // one index block: KG offsets x 128 rows
    constexpr int TMEM_COLS = TILES * COUT < 32 ? 32 : TILES * COUT;
    constexpr uint32_t IDESC = umma_idesc(COUT);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = sA + A_STAGES * A_BYTES;
    int32_t* s_idx = reinterpret_cast<int32_t*>(sB + B_STAGES * B_BYTES);
    float* s_scale = reinterpret_cast<float*>(s_idx + IDX_STAGES * IDX_WORDS);
    float* s_shift = s_scale + COUT;
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(s_shift + COUT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstages = (kvol + KG - 1) / KG;

    if (tid == 0) {
        for (int s = 0; s < A_STAGES; ++s) {
            for (int i = 0; i < MMA_WARPS_MAX; ++i)
                mbar_init(smem_u32(&ctl->a_full[i][s]), 32);   // the lanes of the gather warp that owns the stage
            mbar_init(smem_u32(&ctl->a_empty[s]), 1);
        }
        for (int s = 0; s < B_STAGES; ++s) {
            mbar_init(smem_u32(&ctl->b_full[s]), 1);
            mbar_init(smem_u32(&ctl->b_empty[s]), MMA_WARPS);   // every MMA issuer releases the weight block
        }
        for (int s = 0; s < IDX_STAGES; ++s) {
            mbar_init(smem_u32(&ctl->i_full[s]), 32);
            mbar_init(smem_u32(&ctl->i_empty[s]), 32);
        }
        mbar_init(smem_u32(&ctl->acc_full), MMA_WARPS);        // every MMA issuer reports its tiles
        mbar_init(smem_u32(&ctl->acc_empty), TILE_M);
        mbar_init(smem_u32(&ctl->mma_drain), MMA_WARPS);
        ctl->abort_flag = 0;
        ctl->abort_where = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int c = tid; c < COUT; c += UMMA_THREADS) {
        s_scale[c] = scale ? scale[c] : 1.f;
        s_shift[c] = (scale && shift) ? shift[c] : 0.f;
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;
#ifdef SESSD_UMMA_TIMING
    const long long t_cta0 = clock64();
    unsigned long long tacc[32] = {};   // cycle counters kept in registers, written once at the end
#endif

    const int tiles_per_frame = (max_voxels + TILE_M - 1) / TILE_M;
    uint32_t a_it = 0, b_it = 0, st_it = 0;   // ring positions; every role advances them identically
    uint32_t full_phase = 0;                  // MMA issuers: bit s = parity of the next phase of their a_full[.][s]
    uint32_t b_issued = 0;                    // weight streamer: blocks whose bulk copy has been started

    // Balanced split: the occupied 128-row tiles of all frames, laid end to end, are cut into gridDim.x
    // equal contiguous ranges (row counts are read from the device, so no host round trip); a CTA walks
    // its range in groups of up to TILES tiles of one frame.
    auto frame_rows = [&](int f) {
        const int v = __ldg(out_num + f);
        return v > max_voxels ? max_voxels : (v < 0 ? 0 : v);
    };
    long long total_tiles = 0;
    for (int f = 0; f < batch; ++f) total_tiles += (frame_rows(f) + TILE_M - 1) / TILE_M;
    const int range_lo = (int)(total_tiles * blockIdx.x / gridDim.x);
    const int range_hi = (int)(total_tiles * (blockIdx.x + 1) / gridDim.x);
    int b = 0, frame_first = 0;                 // frame of the cursor and the global index of its first tile
    int n = batch > 0 ? frame_rows(0) : 0;
    int frame_tiles = (n + TILE_M - 1) / TILE_M;

    for (int cur = range_lo; cur < range_hi;) {
        while (cur >= frame_first + frame_tiles) {
            frame_first += frame_tiles;
            ++b;
            n = frame_rows(b);
            frame_tiles = (n + TILE_M - 1) / TILE_M;
        }
        const int tile0 = cur - frame_first;
        int cnt = range_hi - cur;
        cnt = cnt > TILES ? TILES : cnt;
        cnt = cnt > frame_tiles - tile0 ? frame_tiles - tile0 : cnt;
        cur += cnt;
        const int row0 = tile0 * TILE_M;
#ifdef SESSD_UMMA_TIMING
        const long long tg0 = clock64();
#endif
        if (*abort_flag) break;
        uint32_t m[TILES];
        uint32_t any = 0;
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
            m[t] = t < cnt ? __ldg(tile_mask + (size_t)b * tiles_per_frame + tile0 + t) : 0u;
            any |= m[t];
        }
        int n_a = 0, n_b = 0;   // A and B stages this super-tile consumes
        for (int g = 0; g < nstages; ++g) {
            int act = 0;
#pragma unroll
            for (int t = 0; t < TILES; ++t) act += stage_active<KG>(m[t], g) ? 1 : 0;
            n_a += act;
            n_b += act ? 1 : 0;
        }

        if (warp < 4) {
            // ---------------- gather producers ----------------
            // Each of the four gather warps owns every fourth stage and issues all of its copies: while one
            // warp sits in the latency of its barrier hand-offs the other three keep the copy pipe busy.
            // Lane = (row group j, 16-byte chunk c): the eight lanes j*8..j*8+7 copy rows 32j..32j+31 of the
            // stage, one row per step, chunk c of the row landing at chunk c ^ (row & 7) (128-byte swizzle).
            const int c = lane & 7;                // 16-byte chunk of the 128-byte row
            const int jrow = (lane >> 3) * 32;     // first row of this lane group
            const int koff = c / CPO;              // offset of the stage's group this chunk belongs to
            const int csub = (c % CPO) * 8;        // first channel of the chunk
            const __half* in_b = in + (size_t)b * max_voxels * CIN;
            uint32_t my_a = a_it;
#ifdef SESSD_UMMA_TIMING
            const long long tg1 = clock64();
            if (tid == 0 && blockIdx.x < 1) tacc[9] += (unsigned long long)(tg1 - tg0);   // group set-up
#endif
            bool ok = true;
            // list of this group's (stage, tile) pairs: lane g holds stage g's tiles, a warp scan places them
            uint8_t* list = ctl->stage_list[warp];
            {
                const uint32_t bits = lane < nstages ? active_tiles<KG>(m, lane) : 0u;
                const int cnt_l = __popc(bits);
                int incl = cnt_l;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                    if (lane >= d) incl += v;
                }
                int at = incl - cnt_l;
#pragma unroll
                for (int tt = 0; tt < TILES; ++tt)
                    if ((bits >> tt) & 1u) list[at++] = (uint8_t)((lane << 2) | tt);
                __syncwarp();
            }
            const int first = (warp + GATHER_WARPS - (int)(a_it % GATHER_WARPS)) % GATHER_WARPS;
            for (int e = first; e < n_a && ok; e += GATHER_WARPS) {
                my_a = a_it + (uint32_t)e;
                const int code = list[e];
                const int g = code >> 2, t = code & 3;
                const uint32_t s = my_a % A_STAGES, si = my_a % IDX_STAGES;
#ifdef SESSD_UMMA_TIMING
                long long tq0 = clock64();
#endif
                // row indices of this stage, fetched ahead of time by the index warp
                ok = mbar_wait(smem_u32(&ctl->i_full[si]), (my_a / IDX_STAGES) & 1u, abort_flag, 1 | (int)(my_a << 4));
                if (!ok) break;
#ifdef SESSD_UMMA_TIMING
                long long tq1 = clock64();
                long long tq2 = tq1;
#endif
                ok = mbar_wait(smem_u32(&ctl->a_empty[s]), ((my_a / A_STAGES) & 1u) ^ 1u, abort_flag, 2 | (int)(my_a << 4));
                if (!ok) break;
#ifdef SESSD_UMMA_TIMING
                long long tq3 = clock64();
                if (tid == 0 && blockIdx.x < 1 && my_a >= (uint32_t)A_STAGES) {
                    tacc[16] += (unsigned long long)(tq3 - ctl->t_commit[s]);   // commit issued -> stage seen free
                    tacc[17] += 1;
                    if (tq3 - tq2 < 100) tacc[18] += 1;                         // free already when asked
                }
#endif
                const bool k_ok = g * KG + koff < kvol;
                const int rows_left = n - (row0 + t * TILE_M + jrow);   // rows of this lane group inside the frame
                const int32_t* ip = &s_idx[si * IDX_WORDS + koff * TILE_M + jrow];
                const uint32_t a_base = smem_u32(sA + s * A_BYTES) + jrow * ROW_BYTES;
                // Every instruction of this loop is on the critical path of the stage (the gather warps are bound
                // by their own instruction latency, not by the copies), so the common case - all offsets of the
                // stage exist and the whole tile lies inside the frame - takes three instructions per row: a
                // predicate from the sign of the index, the address, and a copy that writes zeros when the
                // predicate says the neighbour is missing.
                const bool plain = g * KG + KG <= kvol && row0 + (t + 1) * TILE_M <= n;   // uniform over the warp
                const __half* lane_base = in_b + csub;
                // all 32 indices first (the copies below are compiler barriers, a load could not move above them)
                int vv[32];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int4 v = *reinterpret_cast<const int4*>(ip + 4 * q);
                    vv[4 * q] = v.x, vv[4 * q + 1] = v.y, vv[4 * q + 2] = v.z, vv[4 * q + 3] = v.w;
                }
                if (plain) {
#pragma unroll
                    for (int p = 0; p < 32; ++p)
                        cp_async_16_or_zero(a_base + p * ROW_BYTES + ((c ^ (p & 7)) << 4),
                                            lane_base + (ptrdiff_t)vv[p] * CIN, vv[p]);
                } else {
#pragma unroll
                    for (int p = 0; p < 32; ++p) {
                        const int id = (k_ok && p < rows_left) ? vv[p] : -1;
                        const __half* src = in_b + (size_t)(id < 0 ? 0 : id) * CIN + csub;
                        cp_async_16(a_base + p * ROW_BYTES + ((c ^ (p & 7)) << 4), src, id < 0 ? 0u : 16u);
                    }
                }
                mbar_arrive(smem_u32(&ctl->i_empty[si]));           // the index block has been read
                // publishes the stage, when the copies land, to the issuer that owns row tile t
                cp_async_arrive_noinc(smem_u32(&ctl->a_full[t & 1][s]));
#ifdef SESSD_UMMA_TIMING
                if (tid == 0 && blockIdx.x < 1) {
                    long long tq5 = clock64();
                    ctl->t_issue[s] = tq5;
                    tacc[0] += (unsigned long long)(tq1 - tq0);  // wait index block
                    tacc[1] += (unsigned long long)(tq3 - tq2);  // wait free A stage
                    tacc[3] += (unsigned long long)(tq5 - tq0);  // whole iteration
                    tacc[4] += 1;
                }
#endif
            }
#ifdef SESSD_UMMA_TIMING
            if (tid == 0 && blockIdx.x < 1) tacc[14] += (unsigned long long)(clock64() - tg1);   // whole gather loop of the group
#endif

            // ---------------- epilogue ----------------
#ifdef SESSD_UMMA_TIMING
            long long te0 = clock64();
#endif
            bool got = true;
            if (any) {
                got = ok && mbar_wait(smem_u32(&ctl->acc_full), st_it & 1u, abort_flag, 3 | (int)(st_it << 4));
                got = __all_sync(0xFFFFFFFFu, got);
                if (got) tc_fence_after();
            }
#ifdef SESSD_UMMA_TIMING
            long long te1 = clock64();
#endif
            // Column blocks of CB channels keep the register footprint small enough for other kernels'
            // blocks to share the SM with the two resident CTAs of this one.
            constexpr int CB = COUT < 32 ? COUT : 32;
#pragma unroll 1
            for (int t2 = 0; t2 < cnt; ++t2) {
                const int row = row0 + t2 * TILE_M + tid;
                const uint32_t m_t2 = t2 == 0 ? m[0] : (t2 == 1 ? m[1] : (t2 == 2 ? m[2] : m[3]));
                const bool have = any && got && m_t2;
                const bool store = got && row < n;
                __half* dst = out + ((size_t)b * max_voxels + row) * COUT;
                __half* d = nullptr;
                if (dense && store) {
                    // fused BEV scatter (sparse2Dense.cu:201-206): channel c*D + z, pixel (y, x)
                    const int4 c4 = __ldg(&out_coors[(size_t)b * max_voxels + row]);
                    d = dense + (size_t)b * COUT * D * H * W + ((size_t)c4.y * H + c4.z) * W + c4.w;
                }
#pragma unroll 1
                for (int cb = 0; cb < COUT; cb += CB) {
                    float acc[CB];
                    if (have) {
#pragma unroll
                        for (int c0 = 0; c0 < CB; c0 += 16) {
                            uint32_t r16[16];
                            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + t2 * COUT + cb + c0, r16);
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[c0 + j] = __uint_as_float(r16[j]);
                        }
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < CB; ++j) acc[j] = 0.f;
                    }
                    if (!store) continue;
#pragma unroll
                    for (int c0 = 0; c0 < CB; c0 += 8) {
                        uint4 pk;
                        __half2* h = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // scale and shift of channels ch, ch+1 as two 8-byte shared-memory reads
                            const int ch = cb + c0 + 2 * j;
                            const float2 sc = *reinterpret_cast<const float2*>(&s_scale[ch]);
                            const float2 sh = *reinterpret_cast<const float2*>(&s_shift[ch]);
                            float v0 = fmaf(acc[c0 + 2 * j], sc.x, sh.x);
                            float v1 = fmaf(acc[c0 + 2 * j + 1], sc.y, sh.y);
                            if (relu) {
                                v0 = v0 > 0.f ? v0 : 0.f;
                                v1 = v1 > 0.f ? v1 : 0.f;
                            }
                            h[j] = __floats2half2_rn(v0, v1);
                        }
                        *reinterpret_cast<uint4*>(dst + cb + c0) = pk;
                        if (d) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                d[(size_t)(cb + c0 + 2 * j) * D * H * W] = __low2half(h[j]);
                                d[(size_t)(cb + c0 + 2 * j + 1) * D * H * W] = __high2half(h[j]);
                            }
                        }
                    }
                }
            }
            if (any) {
                tc_fence_before();
                mbar_arrive(smem_u32(&ctl->acc_empty));   // the accumulators may be overwritten
            }
#ifdef SESSD_UMMA_TIMING
            if (tid == 0 && blockIdx.x < 1) {
                tacc[5] += (unsigned long long)(te1 - te0);          // wait for the accumulators
                tacc[6] += (unsigned long long)(clock64() - te1);    // epilogue proper
                tacc[7] += 1;
            }
#endif
        } else if (warp == 4 || warp == 7) {
            // ---------------- MMA issuers ----------------
            // Issuing a tcgen05.mma or commit costs the issuing thread on the order of a hundred cycles, so
            // two threads issue: warp 4 owns the even row tiles, warp 7 the odd ones (disjoint accumulators;
            // the split stays even when a group holds fewer than TILES tiles).
            if (lane == 0 && any) {
                const int parity = warp == 4 ? 0 : 1;
                uint32_t my_a = a_it, my_b = b_it;
                bool ok = true;
                if (st_it > 0) ok = mbar_wait(smem_u32(&ctl->acc_empty), (st_it - 1u) & 1u, abort_flag, 4 | (int)(st_it << 4));
                if (ok) tc_fence_after();
                uint32_t started = 0;
                for (int g = 0; g < nstages && ok; ++g) {
                    const uint32_t bits = active_tiles<KG>(m, g);
                    const int act = __popc(bits);   // active tiles of this stage group
                    const bool mine = (bits & (parity ? 0xAAAAAAAAu : 0x55555555u)) != 0u;
                    if (!act) continue;
                    const uint32_t sb = my_b % B_STAGES;
                    // Both issuers wait for the block, also one with nothing to do for this group: its
                    // release below must count for this use of the slot, not for an earlier one.
#ifdef SESSD_UMMA_TIMING
                    const long long tb0 = clock64();
#endif
                    ok = mbar_wait(smem_u32(&ctl->b_full[sb]), (my_b / B_STAGES) & 1u, abort_flag, 5 | (int)(my_b << 4));
#ifdef SESSD_UMMA_TIMING
                    if (warp == 4 && blockIdx.x < 1) {
                        tacc[11] += (unsigned long long)(clock64() - tb0);
                    }
#endif
                    if (!ok) break;
                    if (mine) {
                        const uint32_t b_addr = smem_u32(sB + sb * B_BYTES);
                        uint32_t pos = my_a;
                        for (int t = 0; t < TILES && ok; ++t) {
                            if (!((bits >> t) & 1u)) continue;
                            if ((t & 1) != parity) {   // the other issuer's stage
                                ++pos;
                                continue;
                            }
                            const uint32_t sa = pos % A_STAGES;
#ifdef SESSD_UMMA_TIMING
                            const long long tm0 = clock64();
#endif
                            ok = mbar_wait(smem_u32(&ctl->a_full[parity][sa]), (full_phase >> sa) & 1u, abort_flag,
                                           6 | (int)(pos << 4));
                            full_phase ^= 1u << sa;   // this issuer's next use of the slot is the next phase
                            if (!ok) break;
#ifdef SESSD_UMMA_TIMING
                            if (warp == 4 && blockIdx.x < 1) {   // cycles this issuer waited for gathered rows
                                const long long tm1 = clock64();
                                tacc[2] += (unsigned long long)(tm1 - tm0);
                                tacc[19] += (unsigned long long)(tm1 - ctl->t_issue[sa]);   // gathers issued -> seen landed
                                if (tm1 - tm0 < 100) tacc[20] += 1;                          // landed already when asked
                            }
#endif
                            fence_proxy_async();   // the gathered rows were written through the generic proxy
                            tc_fence_after();
                            const uint32_t a_addr = smem_u32(sA + sa * A_BYTES);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk) {
                                umma_f16(tmem + t * COUT, umma_desc(a_addr + kk * 32), umma_desc(b_addr + kk * 32), IDESC,
                                         (((started >> t) & 1u) || kk > 0) ? 1u : 0u);
                            }
                            started |= 1u << t;
                            umma_commit(smem_u32(&ctl->a_empty[sa]));   // frees the A stage once these MMAs have read it
#ifdef SESSD_UMMA_TIMING
                            if (blockIdx.x < 1) ctl->t_commit[sa] = clock64();
                            if (warp == 4 && blockIdx.x < 1) {
                                tacc[10] += (unsigned long long)(clock64() - tm0);   // wait + issue + commit of one stage
                                tacc[12] += 1;
                            }
#endif
                            ++pos;
                        }
                        if (ok) umma_commit(smem_u32(&ctl->b_empty[sb]));
                    } else {
                        mbar_arrive(smem_u32(&ctl->b_empty[sb]));   // nothing to read from this weight block
                    }
                    my_a += act;
                    ++my_b;
                }
                if (ok) {
                    if (started) umma_commit(smem_u32(&ctl->acc_full));
                    else mbar_arrive(smem_u32(&ctl->acc_full));
                }
            }
            __syncwarp();
        } else if (warp == 6) {
            // ---------------- neighbour-index loader ----------------
            // Copies, for every (stage, tile) pair in consumption order, the KG x 128 neighbour indices
            // into the index ring with 4-byte cp.async, several blocks ahead of the gather warps. Rows
            // past max_voxels are zero-filled; the gather warps ignore rows past the frame's row count.
            const int32_t* nbr_b = nbr + (size_t)b * kvol * max_voxels;
            uint32_t my_i = a_it;
            bool ok = true;
            int g = -1, t = 0;
            uint32_t rem = 0;
            while (ok && next_item<KG>(m, nstages, g, rem, t)) {
                const uint32_t si = my_i % IDX_STAGES;
                ok = mbar_wait<true>(smem_u32(&ctl->i_empty[si]), ((my_i / IDX_STAGES) & 1u) ^ 1u, abort_flag, 7 | (int)(my_i << 4));
                if (!ok) break;
#pragma unroll
                for (int j = 0; j < KG; ++j) {
                    const int k = g * KG + j;
#pragma unroll
                    for (int q = 0; q < TILE_M / 32; ++q) {
                        const int r = q * 32 + lane;
                        const int row = row0 + t * TILE_M + r;
                        const bool in_range = k < kvol && row < max_voxels;
                        const int32_t* src = nbr_b + (in_range ? (size_t)k * max_voxels + row : 0);
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(
                                         smem_u32(&s_idx[si * IDX_WORDS + j * TILE_M + r])),
                                     "l"(src), "r"(in_range ? 4u : 0u)
                                     : "memory");
                    }
                }
                cp_async_arrive_noinc(smem_u32(&ctl->i_full[si]));
                ++my_i;
            }
        } else {
            // ---------------- weight streamer ----------------
            if (lane == 0 && !withhold_weights) {
                uint32_t my_b = b_it;
                bool ok = true;
                for (int g = 0; g < nstages && ok; ++g) {
                    bool stage_any = false;
#pragma unroll
                    for (int t = 0; t < TILES; ++t) stage_any |= stage_active<KG>(m[t], g);
                    if (!stage_any) continue;
                    const uint32_t sb = my_b % B_STAGES;
                    ok = mbar_wait<true>(smem_u32(&ctl->b_empty[sb]), ((my_b / B_STAGES) & 1u) ^ 1u, abort_flag, 8 | (int)(my_b << 4));
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&ctl->b_full[sb]);
                    mbar_arrive_expect_tx(bar, B_BYTES);
                    bulk_load(smem_u32(sB + sb * B_BYTES), wtiles + (size_t)g * B_BYTES, B_BYTES, bar);
                    ++my_b;
                    b_issued = my_b;
                }
            }
            __syncwarp();
        }
        a_it += n_a;
        b_it += n_b;
        if (any) ++st_it;
    }

    tc_fence_before();
    __syncthreads();
#ifdef SESSD_UMMA_TIMING
    if ((tid == 0 || tid == 128) && blockIdx.x < 1) {
        unsigned long long* dbg = reinterpret_cast<unsigned long long*>(status) + 96;
        tacc[tid == 0 ? 8 : 13] = (unsigned long long)(clock64() - t_cta0);
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (tacc[i]) dbg[i] = tacc[i];
    }
#endif
    if (*abort_flag) {
        // An aborting CTA must not return while its own copies are still writing shared memory or its MMAs tensor
        // memory: the gather and index warps wait for their cp.async copies, the issuers commit to a barrier that
        // warp 4 waits on (bounded) before it frees the tensor memory, the weight streamer waits (bounded) for
        // its last bulk copies.
        if (warp < GATHER_WARPS || warp == 6) asm volatile("cp.async.wait_all;" ::: "memory");   // rows and indices
        if ((warp == 4 || warp == 7) && lane == 0) umma_commit(smem_u32(&ctl->mma_drain));
        if (warp == 5 && lane == 0) {
            const uint32_t first = b_issued > (uint32_t)B_STAGES ? b_issued - B_STAGES : 0u;
            for (uint32_t j = first; j < b_issued; ++j) {
                const uint32_t bar = smem_u32(&ctl->b_full[j % B_STAGES]);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, (j / B_STAGES) & 1u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
            }
        }
    }
    __syncthreads();
    if (tid == 0 && *abort_flag) {
        atomicOr(status, SESSD_STATUS_TIMEOUT);
        atomicCAS(status + 1, 0, ctl->abort_where);   // first report wins: which wait, at which ring position
    }
    if (warp == 4) {
        if (*abort_flag && lane == 0) {
            // the tensor memory is given back only when no MMA of this CTA can still write to it
            const long long t0 = clock64();
            while (!mbar_try_wait(smem_u32(&ctl->mma_drain), 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int CIN, int COUT>
int launch_one(const ConvLaunch& c, cudaStream_t stream) {
    static const std::string name = "conv_umma<f16," + std::to_string(CIN) + "," + std::to_string(COUT) + ">";
    constexpr int ctas_per_sm = 2;   // shared memory and registers are budgeted for two resident CTAs
    const int smem = umma_smem_bytes<CIN, COUT>();
    // the attribute belongs to the device's context: set it once per device (repeating it is harmless, so a
    // race between two host threads only costs a second call)
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    SESSD_CUDA(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        SESSD_CUDA(cudaFuncSetAttribute(conv_umma_kernel<CIN, COUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    SESSD_LAUNCH_NAMED(name.c_str(), (conv_umma_kernel<CIN, COUT>), persistent_grid(ctas_per_sm), UMMA_THREADS, smem, stream,
                       static_cast<const __half*>(c.in), static_cast<__half*>(c.out), c.nbr, c.tile_mask, c.out_num,
                       static_cast<const uint8_t*>(c.umma_weights), c.scale, c.shift, c.relu, c.batch, c.max_voxels,
                       c.kvol, static_cast<__half*>(c.dense), reinterpret_cast<const int4*>(c.out_coors), c.D, c.H, c.W,
                       c.status, c.debug_withhold_weights);
    return SESSD_OK;
}

}  // namespace

bool conv_umma_supported(int cin, int cout) {
    return (cin == 16 || cin == 32 || cin == 64) && (cout == 16 || cout == 32 || cout == 64);
}

// Weight tiles in the order the kernel consumes them: for stage g (a group of 64/Cin kernel offsets) a
// block of Cout rows x 128 bytes, row n holding K index kk = j*Cin + ci -> W[g*KG + j][ci][n], stored
// K-major with the 128-byte swizzle (16-byte chunk index XOR row index mod 8), zero beyond kvol.
int conv_umma_pack_weights(const float* weights, int kvol, int cin, int cout, void** device_out) {
    *device_out = nullptr;
    if (!conv_umma_supported(cin, cout)) return SESSD_OK;
    const int kg = 64 / cin, nstages = (kvol + kg - 1) / kg;
    std::vector<__half> img((size_t)nstages * cout * 64, __float2half_rn(0.f));
    for (int g = 0; g < nstages; ++g)
        for (int n = 0; n < cout; ++n)
            for (int kk = 0; kk < 64; ++kk) {
                const int k = g * kg + kk / cin, ci = kk % cin;
                if (k >= kvol) continue;
                const int chunk = kk / 8;
                const size_t pos = ((size_t)g * cout + n) * 64 + (size_t)((chunk ^ (n & 7)) * 8) + (kk % 8);
                img[pos] = __float2half_rn(weights[((size_t)k * cin + ci) * cout + n]);
            }
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, img.size() * sizeof(__half));
    if (e == cudaSuccess) e = cudaMemcpy(d, img.data(), img.size() * sizeof(__half), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        set_cuda_error(e, "conv_umma_pack_weights");
        if (d) cudaFree(d);
        return SESSD_ERR_CUDA;
    }
    *device_out = d;
    return SESSD_OK;
}

int launch_conv_umma(const ConvLaunch& c, cudaStream_t stream) {
    if (c.dtype != SESSD_F16 || !c.umma_weights || !c.tile_mask || c.kvol > KVOL_MAX) return SESSD_ERR_UNSUPPORTED;
#define SESSD_CASE(CI, CO) \
    if (c.cin == CI && c.cout == CO) return launch_one<CI, CO>(c, stream);
    SESSD_CASE(16, 16)
    SESSD_CASE(16, 32)
    SESSD_CASE(32, 32)
    SESSD_CASE(32, 64)
    SESSD_CASE(64, 64)
#undef SESSD_CASE
    return SESSD_ERR_UNSUPPORTED;
}

}  // namespace sessd
