// Sparse convolution as an implicit GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces, for fp16 features and 16/32/64 channels, the reference's per-offset scalar kernel
// (submConv3dlayer.cu:479-518, launched kvol times per layer, :632-638). A tile is 128 output rows. For
// every group of kernel offsets ("stage": 64/Cin offsets side by side) the 128 neighbour rows are gathered
// into shared memory as a K-major, 128-byte-swizzled A operand (one 128-byte row per output row, missing
// neighbours zero-filled), the matching pre-tiled weight block is streamed in as the B operand with a bulk
// asynchronous copy, and tcgen05.mma (M = 128, N = Cout, K = 16 x 4) accumulates into an fp32 accumulator in
// tensor memory that stays resident across all offsets. A CTA iteration ("group") covers four tiles with
// the offset loop outermost, so that a weight block is fetched once per four tiles; (tile, stage) pairs
// without any neighbour are skipped using the per-tile offset masks the rulebook kernels produce. The
// epilogue reads the accumulator with tcgen05.ld, applies the folded BatchNorm scale/shift and ReLU, and
// stores fp16 rows (and, for the last layer, scatters them into the dense BEV map).
//
// One persistent CTA per SM; every role has warps of its own and walks the same sequence of groups:
//   warps 0-3    epilogue (warp w reads tensor-memory lanes 32w .. 32w+31). The accumulators are double
//                buffered (2 sets x 4 tiles x Cout columns), so the epilogue of one group runs while the
//                other roles are already working on the next group. A thread holds one row; the rows go
//                through a small staging area of the warp, so that a store instruction writes whole 32- or
//                64-byte runs of 8 or 16 rows instead of one 16-byte piece of 32 rows (those piecemeal
//                stores alone were an eighth of the kernel's time).
//   warps 4-7    MMA issuers; issuer t owns tile t of every group. The warp works out the group's schedule
//                once (lane g for stage g) and walks it together; one elected lane issues the tcgen05.mma and
//                commit instructions (each costs its thread on the order of a hundred cycles, so four share).
//   warp  8      streams the weight blocks (cp.async.bulk) into a three-slot ring.
//   warp  9      prefetches the neighbour indices of upcoming (tile, stage) items into a ring of index blocks
//                with bulk copies, sixteen items side by side (one lane each), two to three slot cycles ahead.
//   warps 10..   gather. The A ring has one 16 KB slot per gather warp: item q (the q-th (tile, stage) pair
//                of the CTA's life) lives in slot q % NSLOT and is filled by warp q % NSLOT alone with
//                sixteen-byte cp.async copies that publish the slot themselves (mbarrier arrival of the
//                copies). With ten slots in flight the latency chain of one slot (issue, landing, MMA,
//                commit) is covered and no barrier is shared between gather warps.
// Every barrier has one waiting role that sees each of its phases in order (a parity wait is only safe
// then): a_full exists per (issuer, slot); index block j is always read by gather warp j % NSLOT.
// A CTA walks a contiguous range of the occupied row tiles, cut so that every CTA gets the same number of
// (tile, stage) items (row counts and masks are read on the device). Every wait is bounded by a clock limit,
// after which the CTA raises SESSD_STATUS_TIMEOUT (and reports which wait in the status block), stops issuing
// work, waits for its own copies and MMAs, frees its tensor memory and returns.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace sessd {

namespace {

constexpr int TILE_M = 128;
constexpr int TILES = 4;                     // row tiles per group; they share each weight block
constexpr int EPI_WARPS = 4;                 // warps 0-3
constexpr int MMA_WARPS = TILES;             // warps 4-7: issuer t owns tile t
constexpr int WEIGHT_WARP = EPI_WARPS + MMA_WARPS;
constexpr int INDEX_WARP = WEIGHT_WARP + 1;
constexpr int FIRST_GATHER_WARP = INDEX_WARP + 1;
constexpr int NSLOT_MAX = 12;
constexpr int NIDX_MAX = 36;
constexpr int B_STAGES = 3;                  // weight ring: a group needs up to 27 blocks, each an L2 round trip away
constexpr int ROW_BYTES = 128;               // 64 halves per A/B row
constexpr int A_BYTES = TILE_M * ROW_BYTES;  // 16 KB
constexpr int KVOL_MAX = 27;
// Words from one offset's 128 indices to the next offset's inside an index block: 16 bytes more than the indices
// take, so that lanes reading different offsets of a stage (32- and 16-channel inputs) use different banks too.
constexpr int TAP_WORDS = kNbrRun;
static_assert(kNbrRun == TILE_M + 4, "the map's spacing between offsets is the index block's");
constexpr long long WAIT_LIMIT_CYCLES = 200000000LL;   // about a tenth of a second; real waits are microseconds

// Gather slots (= gather warps): as many as fit beside the weight ring, the index blocks and the epilogue's staging area.
// The index ring is deeper than the A ring (index rows come from DRAM, several microseconds away under load):
// block j = q % NIDX, with NIDX a multiple of NSLOT so that block j is always read by gather warp j % NSLOT.
template <int CIN>
struct Ring {
    static constexpr int NSLOT = 10;
    static constexpr int NIDX = (CIN == 16 ? 2 : 3) * NSLOT;
    static constexpr int THREADS = (FIRST_GATHER_WARP + NSLOT) * 32;
};

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
// polls). RELAXED waits (roles with slack: weight and index prefetch) also sleep between polls. The MMA
// issuers use the plain limit, every other role one and a half times that: when something upstream is
// missing, the wait closest to the cause is the one that gets reported.
template <bool RELAXED = false, bool ISSUER = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    const long long limit = ISSUER ? WAIT_LIMIT_CYCLES : WAIT_LIMIT_CYCLES + WAIT_LIMIT_CYCLES / 2;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (RELAXED) __nanosleep(200);
            if (mbar_try_wait_parked(bar, parity, 1000u)) return true;
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            if (*abort_flag == 0) abort_flag[1] = where;   // abort_where follows abort_flag in SharedCtl
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// 16-byte copy that writes zeros instead when index < 0 (the source address is then not touched), and
// nothing at all when `was_zero` is set as well: the destination still holds the zeros an earlier copy wrote.
__device__ __forceinline__ void cp_async_16_or_zero_once(uint32_t dst, const void* src, int index, uint32_t was_zero) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.lt.s32 p, %2, 0;\n\t"
        "setp.ne.and.b32 q, %3, 0, p;\n\t"
        "@!q cp.async.cg.shared.global [%0], [%1], 16, p;\n\t}" ::"r"(dst),
        "l"(src), "r"(index), "r"(was_zero)
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
// descriptor version 1, layout type 2 (SWIZZLE_128B). The start address sits in the low 14 bits in units
// of 16 bytes, so stepping 32 bytes along K adds 2 to the descriptor.
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

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct SharedCtl {
    // a_full[t][s]: slot s has landed, for the issuer of tile t. One barrier per (issuer, slot) keeps a single
    // waiter per barrier: parity waits are only safe when the waiter has itself seen every earlier phase.
    unsigned long long a_full[MMA_WARPS][NSLOT_MAX];
    unsigned long long a_empty[NSLOT_MAX];   // the MMAs that read slot s have completed (commit of its issuer)
    unsigned long long i_full[NIDX_MAX];     // index block j has landed
    unsigned long long i_empty[NIDX_MAX];    // gather warp j % NSLOT has read index block j
    unsigned long long b_full[B_STAGES];
    unsigned long long b_empty[B_STAGES];    // every issuer has released the block (commit of its MMAs, or a plain arrival)
    unsigned long long acc_full[2];          // every issuer has committed its tile of the group (per accumulator set)
    unsigned long long acc_empty[2];         // the epilogue has read the set
    unsigned long long mma_drain;            // aborting CTA only: completes when the issuers' outstanding MMAs have finished
    uint32_t tmem_base;
    int abort_flag;
    int abort_where;   // code of the first wait that ran out (role and ring position), for the status block
    // per gather warp: the (stage << 2 | tile) codes of the current group's items in ring order, so that a warp
    // steps straight to the items it owns
    uint8_t stage_list[NSLOT_MAX][TILES * 32];
    uint8_t idx_list[TILES * 32];            // the same list for the index warp
    uint32_t scan_warp[32];                  // work split: per-warp totals of the block scan
    int range_lo, range_hi;                  // work split: this CTA's tiles
    uint32_t idx_uses[NIDX_MAX];             // bulk copies issued into index block j so far (for the abort path)
};

// Epilogue staging: every epilogue warp owns room for its 32 rows of one column block (up to 32 channels), so that
// the rows leave for global memory as whole 32- or 64-byte runs instead of one 16-byte piece per row and store.
template <int COUT>
__host__ __device__ constexpr int stage_row_bytes() { return (COUT < 32 ? COUT : 32) * 2; }
template <int COUT>
__host__ __device__ constexpr int stage_bytes() { return EPI_WARPS * 32 * stage_row_bytes<COUT>(); }

template <int CIN, int COUT>
constexpr int umma_smem_bytes() {
    return 1024 /*alignment slack*/ + Ring<CIN>::NSLOT * A_BYTES + B_STAGES * COUT * ROW_BYTES +
           Ring<CIN>::NIDX * (64 / CIN) * TAP_WORDS * 4 + stage_bytes<COUT>() + (int)sizeof(SharedCtl);
}

// Offsets g*KG .. g*KG+KG-1 of a tile's 27-bit offset mask.
template <int KG>
__device__ __forceinline__ bool stage_active(uint32_t kmask, int g) {
    return ((kmask >> (g * KG)) & ((1u << KG) - 1u)) != 0u;
}

// One bit per stage (at bit position g * KG) that is set when the tile has a neighbour under any offset of the stage.
template <int KG>
__device__ __forceinline__ uint32_t stage_bits(uint32_t kmask) {
    if (KG == 1) return kmask;
    if (KG == 2) return (kmask | (kmask >> 1)) & 0x55555555u;
    uint32_t v = kmask | (kmask >> 1);
    v |= v >> 2;
    return v & 0x11111111u;
}

// Bit t set when row tile t has a neighbour under the offsets of stage g. The masks are only ever indexed
// with compile-time constants, so they stay in registers.
template <int KG>
__device__ __forceinline__ uint32_t active_tiles(const uint32_t (&m)[TILES], int g) {
    uint32_t bits = 0;
#pragma unroll
    for (int t = 0; t < TILES; ++t) bits |= (stage_active<KG>(m[t], g) ? 1u : 0u) << t;
    return bits;
}

// Advances to the next (stage g, tile t) item with work, in the order stage-major, tile-minor; `rem` holds
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

// Folded batch-norm scale and shift of the layer as launch parameters: the epilogue's multiply-adds then take them
// straight from the constant bank (its column loops are unrolled, so every index is a constant), where the
// earlier shared-memory copies cost two loads per channel pair and row on the pipe the gather copies keep busy.
struct EpiConst {
    float scale[64];
    float shift[64];
};

// Lane g holds `bits`, the tiles with work under stage g. Returns the number of (tile, stage) items of the stages
// before g and, in blocks_before, the number of those stages that have any work. Five warp votes: a vote answers
// in a few cycles, while a shuffle scan (five to ten shuffles, each a trip through the shared-memory pipe that the
// gather copies keep busy) cost every role some thousand cycles at each group boundary.
__device__ __forceinline__ int items_before_stage(uint32_t bits, int lane, int* blocks_before = nullptr) {
    const uint32_t lt = (1u << lane) - 1u;
    int items = 0;
#pragma unroll
    for (int t = 0; t < TILES; ++t) items += __popc(__ballot_sync(0xFFFFFFFFu, (bits >> t) & 1u) & lt);
    if (blocks_before) *blocks_before = __popc(__ballot_sync(0xFFFFFFFFu, bits != 0u) & lt);
    return items;
}

template <int CIN, int COUT>
__global__ void __launch_bounds__(Ring<CIN>::THREADS, 1)
conv_umma_kernel(const __half* __restrict__ in, __half* __restrict__ out, const int32_t* __restrict__ nbr,
                 const uint32_t* __restrict__ tile_mask, const int32_t* __restrict__ out_num,
                 const uint8_t* __restrict__ wtiles, const __grid_constant__ EpiConst epi, int relu, int batch,
                 int max_voxels, int kvol, __half* __restrict__ dense, const int4* __restrict__ out_coors, int D, int H,
                 int W, int32_t* status, int withhold_weights) {
    // withhold_weights (tests of the time-out path only): the weight streamer stays silent, so the MMA issuers'
    // bounded wait for the first weight block runs out and every CTA with work leaves through the abort path.
    constexpr int KG = 64 / CIN;            // kernel offsets sharing one 128-byte A row
    constexpr int CPO = CIN / 8;            // 16-byte chunks per offset
    constexpr int B_BYTES = COUT * ROW_BYTES;
    constexpr int NSLOT = Ring<CIN>::NSLOT;
    constexpr int NIDX = Ring<CIN>::NIDX;
    constexpr int THREADS = Ring<CIN>::THREADS;
    constexpr int IDX_WORDS = KG * TAP_WORDS;  // one index block: KG offsets x 128 rows
    constexpr int IDX_BATCH = 16;           // items the index warp handles side by side (must stay below NIDX)
    constexpr int SET_COLS = TILES * COUT;  // accumulator columns of one set
    constexpr int TMEM_COLS = 2 * SET_COLS < 32 ? 32 : 2 * SET_COLS;
    constexpr uint32_t IDESC = umma_idesc(COUT);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = sA + NSLOT * A_BYTES;
    int32_t* s_idx = reinterpret_cast<int32_t*>(sB + B_STAGES * B_BYTES);
    uint8_t* s_stage = reinterpret_cast<uint8_t*>(s_idx + NIDX * IDX_WORDS);
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(s_stage + stage_bytes<COUT>());

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nstages = (kvol + KG - 1) / KG;

    if (tid == 0) {
        for (int s = 0; s < NSLOT; ++s) {
            for (int i = 0; i < MMA_WARPS; ++i)
                mbar_init(smem_u32(&ctl->a_full[i][s]), 32);   // the lanes of the gather warp that owns the slot
            mbar_init(smem_u32(&ctl->a_empty[s]), 1);
        }
        for (int j = 0; j < NIDX; ++j) {
            ctl->idx_uses[j] = 0;
            mbar_init(smem_u32(&ctl->i_full[j]), 1);           // the lane of the index warp that issues the block's copy
            mbar_init(smem_u32(&ctl->i_empty[j]), 32);         // the lanes of the gather warp
        }
        for (int s = 0; s < B_STAGES; ++s) {
            mbar_init(smem_u32(&ctl->b_full[s]), 1);
            mbar_init(smem_u32(&ctl->b_empty[s]), MMA_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&ctl->acc_full[s]), MMA_WARPS);          // every MMA issuer reports its tile
            mbar_init(smem_u32(&ctl->acc_empty[s]), EPI_WARPS * 32);    // every epilogue thread
        }
        mbar_init(smem_u32(&ctl->mma_drain), MMA_WARPS);
        ctl->abort_flag = 0;
        ctl->abort_where = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int tiles_per_frame = (max_voxels + TILE_M - 1) / TILE_M;
    if (warp == EPI_WARPS) {
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
    const bool leader = elect_one();   // one lane per warp, the same one for the whole kernel

    uint32_t a_it = 0, b_it = 0, acc_it = 0;  // items, weight blocks and accumulator sets used so far; every role advances them identically
    uint32_t full_phase = 0;                  // MMA issuers: bit s = parity of the next phase of their a_full[t][s]
    uint32_t b_issued = 0;                    // weight streamer: blocks whose bulk copy has been started
    uint32_t zero_rows = 0;                   // gather warps: bit p = this lane's chunk of row p of its slot holds zeros

    // Balanced split: the occupied 128-row tiles of all frames, laid end to end, are cut into gridDim.x
    // contiguous ranges of equal work (row counts and tile masks are read from the device, so no host round
    // trip); a CTA walks its range in groups of up to TILES tiles of one frame. The work of a tile is the number
    // of its (tile, stage) items plus a constant for its epilogue: rows numbered in spatial order make
    // neighbouring tiles alike, so dense and sparse regions would otherwise load the CTAs unevenly.
    // Every CTA computes the same cut points from the same masks: thread t sums the weights of its slice of the
    // tile sequence, a block scan turns the sums into running totals, and the threads whose slice holds cut
    // point blockIdx.x or blockIdx.x + 1 walk the slice to the tile where the running total passes the target.
    auto frame_rows = [&](int f) {
        const int v = __ldg(out_num + f);
        return v > max_voxels ? max_voxels : (v < 0 ? 0 : v);
    };
    int total_tiles = 0;
    for (int f = 0; f < batch; ++f) total_tiles += (frame_rows(f) + TILE_M - 1) / TILE_M;
    {
        const int per = (total_tiles + THREADS - 1) / THREADS;
        const int first = tid * per, last = first + per < total_tiles ? first + per : total_tiles;
        // a tile costs its items plus its share of the group hand-over and of the epilogue, about eight items' worth
        // (fitted to the CTA lifetimes of 1/4-resolution launches)
        auto tile_weight = [&](uint32_t mask) { return (uint32_t)(__popc(stage_bits<KG>(mask)) + 8); };
        int f = 0, f_first = 0, f_tiles = batch > 0 ? (frame_rows(0) + TILE_M - 1) / TILE_M : 0;
        auto seek = [&](int tile) {   // frame of a tile of the sequence (tiles are visited in ascending order)
            while (f < batch && tile >= f_first + f_tiles) {
                f_first += f_tiles;
                ++f;
                f_tiles = f < batch ? (frame_rows(f) + TILE_M - 1) / TILE_M : 0;
            }
        };
        uint32_t mine = 0;
        for (int i = first; i < last; ++i) {
            seek(i);
            mine += tile_weight(__ldg(tile_mask + (size_t)f * tiles_per_frame + (i - f_first)));
        }
        uint32_t incl = mine;   // inclusive block scan of `mine`
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += v;
        }
        if (lane == 31) ctl->scan_warp[warp] = incl;
        if (tid == 0) ctl->range_lo = 0, ctl->range_hi = total_tiles;
        __syncthreads();
        uint32_t before = 0, grand = 0;
        for (int w = 0; w < THREADS / 32; ++w) {
            const uint32_t v = ctl->scan_warp[w];
            if (w < warp) before += v;
            grand += v;
        }
        const uint32_t excl = before + incl - mine;   // weight of all tiles before this thread's slice
        // cut point c: the first tile whose running total (inclusive) exceeds grand * c / gridDim.x
        for (int side = 0; side < 2; ++side) {
            const unsigned long long c = blockIdx.x + side;
            if (c == 0 || c >= gridDim.x) continue;   // 0 and total_tiles are preset
            const uint32_t target = (uint32_t)((unsigned long long)grand * c / gridDim.x);
            if (mine == 0 || target < excl || target >= excl + mine) continue;
            f = 0, f_first = 0, f_tiles = batch > 0 ? (frame_rows(0) + TILE_M - 1) / TILE_M : 0;
            uint32_t run = excl;
            int cut = last;
            for (int i = first; i < last; ++i) {
                seek(i);
                run += tile_weight(__ldg(tile_mask + (size_t)f * tiles_per_frame + (i - f_first)));
                if (run > target) {
                    cut = i;
                    break;
                }
            }
            if (side == 0) ctl->range_lo = cut;
            else ctl->range_hi = cut;
        }
    }
    __syncthreads();
    const int range_lo = ctl->range_lo, range_hi = ctl->range_hi;
    // The walk is one group ahead of the work: the masks of the next group are requested when the current group
    // starts, so that no role sits in the latency of those reads at a group boundary (every role of the CTA would
    // stall there at about the same time and drain the pipeline).
    int c_b = 0, c_first = 0;                   // cursor: frame and the global index of its first tile
    int c_n = batch > 0 ? frame_rows(0) : 0;
    int c_tiles = (c_n + TILE_M - 1) / TILE_M;
    int c_cur = range_lo;
    int nx_b = 0, nx_n = 0, nx_tile0 = 0, nx_cnt = 0;   // the next group
    uint32_t nx_m[TILES] = {0u, 0u, 0u, 0u};
    auto fetch_next = [&]() {
        nx_cnt = 0;
        if (c_cur >= range_hi) return;
        while (c_cur >= c_first + c_tiles) {
            c_first += c_tiles;
            ++c_b;
            c_n = frame_rows(c_b);
            c_tiles = (c_n + TILE_M - 1) / TILE_M;
        }
        nx_b = c_b;
        nx_n = c_n;
        nx_tile0 = c_cur - c_first;
        int cnt = range_hi - c_cur;
        cnt = cnt > TILES ? TILES : cnt;
        cnt = cnt > c_tiles - nx_tile0 ? c_tiles - nx_tile0 : cnt;
        nx_cnt = cnt;
        c_cur += cnt;
#pragma unroll
        for (int t = 0; t < TILES; ++t)
            nx_m[t] = t < cnt ? __ldg(tile_mask + (size_t)nx_b * tiles_per_frame + nx_tile0 + t) : 0u;
    };
    fetch_next();

    while (nx_cnt > 0) {
        const int b = nx_b, n = nx_n, tile0 = nx_tile0, cnt = nx_cnt;
        const int row0 = tile0 * TILE_M;
        uint32_t m[TILES];
        uint32_t any = 0;
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
            m[t] = nx_m[t];
            any |= m[t];
        }
        fetch_next();   // reads issued now, used at the top of the next iteration
        if (*abort_flag) break;
        // items and weight blocks this group consumes
        const uint32_t sb0 = stage_bits<KG>(m[0]), sb1 = stage_bits<KG>(m[1]), sb2 = stage_bits<KG>(m[2]),
                       sb3 = stage_bits<KG>(m[3]);
        const int n_a = __popc(sb0) + __popc(sb1) + __popc(sb2) + __popc(sb3);
        const int n_b = __popc(sb0 | sb1 | sb2 | sb3);
        const uint32_t set = acc_it & 1u;           // accumulator set of this group (groups without work use none)
        const uint32_t set_phase = (acc_it >> 1) & 1u;

        if (warp >= FIRST_GATHER_WARP) {
            // ---------------- gather producers ----------------
            // Gather warp s fills slot s with every NSLOT-th item and issues all of its copies: while one warp
            // sits in the latency of its barrier hand-offs the others keep the copy pipe busy.
            // Lane = (row group j, 16-byte chunk c): the eight lanes j*8..j*8+7 copy, in step p, chunk c of row
            // 32 (p / 8) + 8 j + p % 8 of the item to chunk c ^ (row & 7) of the slot's row (128-byte swizzle).
            // With the rows of a group in runs of eight, the four groups' 16-byte index reads of one instruction
            // lie 32 bytes apart (different banks: one pass), where runs of 32 rows put them 128 bytes apart
            // (the same banks: four passes).
            const int s = warp - FIRST_GATHER_WARP;
            const int c = lane & 7;                // 16-byte chunk of the 128-byte row
            const int jrow = (lane >> 3) * 8;      // first row of this lane group's first run of eight
            const int koff = c / CPO;              // offset of the stage's group this chunk belongs to
            const int csub = (c % CPO) * 8;        // first channel of the chunk
            const __half* in_b = in + (size_t)b * max_voxels * CIN;
            // list of this group's items: lane g holds stage g's tiles, a warp scan places them
            uint8_t* list = ctl->stage_list[s];
            {
                const uint32_t bits = lane < nstages ? active_tiles<KG>(m, lane) : 0u;
                int at = items_before_stage(bits, lane);
#pragma unroll
                for (int tt = 0; tt < TILES; ++tt)
                    if ((bits >> tt) & 1u) list[at++] = (uint8_t)((lane << 2) | tt);
                __syncwarp();
            }
            const int first = (s + NSLOT - (int)(a_it % NSLOT)) % NSLOT;
            const uint32_t idx_lane = smem_u32(&s_idx[koff * TAP_WORDS + jrow]);
            const uint32_t a_base = smem_u32(sA + s * A_BYTES) + jrow * ROW_BYTES;
            for (int e = first; e < n_a; e += NSLOT) {
                const uint32_t q = a_it + (uint32_t)e;
                const uint32_t use = (q / NSLOT) & 1u;   // parity of this use of the slot
                const uint32_t ji = q % NIDX;            // index block of the item
                const uint32_t iuse = (q / NIDX) & 1u;
                const uint32_t idx_base = idx_lane + ji * (IDX_WORDS * 4);
                const int code = list[e];
                const int g = code >> 2, t = code & 3;
                // row indices of this item, fetched ahead of time by the index warp
                if (!mbar_wait(smem_u32(&ctl->i_full[ji]), iuse, abort_flag, 1 | (int)(q << 4))) break;

                // all 32 indices first (the copies below are compiler barriers, a load could not move above them)
                int vv[32];
#pragma unroll
                for (int w4 = 0; w4 < 8; ++w4) {
                    int4 v;
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                 : "r"(idx_base + 128 * (w4 >> 1) + 16 * (w4 & 1)));   // rows 32 (w4 / 2) + 8 j + 4 (w4 % 2) ..
                    vv[4 * w4] = v.x, vv[4 * w4 + 1] = v.y, vv[4 * w4 + 2] = v.z, vv[4 * w4 + 3] = v.w;
                }
                if (!mbar_wait(smem_u32(&ctl->a_empty[s]), use ^ 1u, abort_flag, 2 | (int)(q << 4))) break;
                const bool k_ok = g * KG + koff < kvol;
                const int rows_left = n - (row0 + t * TILE_M + jrow);   // step p's row lies inside the frame when 32 (p / 8) + p % 8 < rows_left
                // Every instruction of this loop is on the critical path of the item, so the common case - all
                // offsets of the stage exist and the whole tile lies inside the frame - takes three instructions
                // per row: a predicate from the sign of the index, the address, and a copy that writes zeros when
                // the predicate says the neighbour is missing.
                const bool plain = g * KG + KG <= kvol && row0 + (t + 1) * TILE_M <= n;   // uniform over the warp
                const __half* lane_base = in_b + csub;
                if (plain) {
                    // More than half of an item's rows are missing neighbours, and a third are missing in two
                    // consecutive uses of the slot: their zeros are still there, so the copy is left out (the
                    // shared-memory write of a zero row costs the same as that of a real one).
                    uint32_t zero_now = 0;
#pragma unroll
                    for (int p = 0; p < 32; ++p) {
                        cp_async_16_or_zero_once(a_base + (32 * (p >> 3) + (p & 7)) * ROW_BYTES + ((c ^ (p & 7)) << 4),
                                                 lane_base + (ptrdiff_t)vv[p] * CIN, vv[p], zero_rows & (1u << p));
                        zero_now |= ((uint32_t)vv[p] >> 31) << p;
                    }
                    zero_rows = zero_now;
                } else {
                    zero_rows = 0;   // (the general path writes every row)
#pragma unroll
                    for (int p = 0; p < 32; ++p) {
                        const int id = (k_ok && 32 * (p >> 3) + (p & 7) < rows_left) ? vv[p] : -1;
                        const __half* src = in_b + (size_t)(id < 0 ? 0 : id) * CIN + csub;
                        cp_async_16(a_base + (32 * (p >> 3) + (p & 7)) * ROW_BYTES + ((c ^ (p & 7)) << 4), src,
                                    id < 0 ? 0u : 16u);
                    }
                }
                // The index block may be refilled now: every index has been consumed by a copy above (the arrival
                // sits behind the copies so that it depends on the registers the index loads wrote; released
                // earlier, right after the loads were issued, the last of them were seen to return the next
                // item's indices). The ring is three slot cycles deep, so nothing waits for this.
                mbar_arrive(smem_u32(&ctl->i_empty[ji]));
                // publishes the slot, when the copies land, to the issuer that owns row tile t
                cp_async_arrive_noinc(smem_u32(&ctl->a_full[t][s]));
            }
        } else if (warp < EPI_WARPS) {
            // ---------------- epilogue ----------------
            bool got = true;
            if (any) {
                got = mbar_wait<true>(smem_u32(&ctl->acc_full[set]), set_phase, abort_flag, 3 | (int)(acc_it << 4));
                got = __all_sync(0xFFFFFFFFu, got);
                if (got) tc_fence_after();
            }
            // Column blocks of CB channels keep the register footprint small.
            constexpr int CB = COUT < 32 ? COUT : 32;
            constexpr int RB = stage_row_bytes<COUT>();   // bytes of a row's column block
            constexpr int CPR = RB / 16;                  // 16-byte chunks per row and block: 4 or 2
            uint8_t* stage = s_stage + warp * (32 * RB);
            auto stage_swz = [](int r) { return RB == 64 ? (r >> 1) & 3 : (r >> 2) & 1; };
#pragma unroll 1
            for (int t2 = 0; t2 < cnt; ++t2) {
                const int row = row0 + t2 * TILE_M + tid;
                const uint32_t m_t2 = t2 == 0 ? m[0] : (t2 == 1 ? m[1] : (t2 == 2 ? m[2] : m[3]));
                const bool have = any && got && m_t2;
                const bool store = got && row < n;
                __half* d = nullptr;
                if (dense && store) {
                    // fused BEV scatter (sparse2Dense.cu:201-206): channel c*D + z, pixel (y, x)
                    const int4 c4 = __ldg(&out_coors[(size_t)b * max_voxels + row]);
                    d = dense + (size_t)b * COUT * D * H * W + ((size_t)c4.y * H + c4.z) * W + c4.w;
                }
#pragma unroll
                for (int cb = 0; cb < COUT; cb += CB) {
                    float acc[CB];
                    if (have) {
                        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + set * SET_COLS + t2 * COUT + cb;
                        if constexpr (CB == 32) {
                            uint32_t r32[32];
                            tmem_ld32(taddr, r32);
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r32[j]);
                        } else {
                            uint32_t r16[16];
                            tmem_ld16(taddr, r16);
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(r16[j]);
                        }
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < CB; ++j) acc[j] = 0.f;
                    }
                    // Every lane packs its row's block into the warp's staging area (16-byte chunks XOR-swizzled by
                    // row so that neither the writes nor the reads below meet in a bank) ...
#pragma unroll
                    for (int c0 = 0; c0 < CB; c0 += 8) {
                        uint4 pk;
                        __half2* h = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int ch = cb + c0 + 2 * j;   // a constant after unrolling
                            float v0 = fmaf(acc[c0 + 2 * j], epi.scale[ch], epi.shift[ch]);
                            float v1 = fmaf(acc[c0 + 2 * j + 1], epi.scale[ch + 1], epi.shift[ch + 1]);
                            if (relu) {
                                v0 = v0 > 0.f ? v0 : 0.f;
                                v1 = v1 > 0.f ? v1 : 0.f;
                            }
                            h[j] = __floats2half2_rn(v0, v1);
                        }
                        *reinterpret_cast<uint4*>(stage + lane * RB + (((c0 >> 3) ^ stage_swz(lane)) << 4)) = pk;
                        if (d) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                d[(size_t)(cb + c0 + 2 * j) * D * H * W] = __low2half(h[j]);
                                d[(size_t)(cb + c0 + 2 * j + 1) * D * H * W] = __high2half(h[j]);
                            }
                        }
                    }
                    __syncwarp();
                    // ... and the warp copies the block out with CPR lanes per row: each store instruction writes
                    // 32 / CPR rows as whole runs of RB bytes.
                    if (got) {
#pragma unroll
                        for (int i = 0; i < CPR; ++i) {
                            const int rr = lane / CPR + i * (32 / CPR), cc = lane % CPR;
                            const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * RB + ((cc ^ stage_swz(rr)) << 4));
                            const int grow = row0 + t2 * TILE_M + warp * 32 + rr;
                            if (grow < n)
                                *reinterpret_cast<uint4*>(out + ((size_t)b * max_voxels + grow) * COUT + cb + cc * 8) = v;
                        }
                    }
                    __syncwarp();
                }
            }
            if (any && got) {
                tc_fence_before();
                mbar_arrive(smem_u32(&ctl->acc_empty[set]));   // the set may be overwritten
            }
        } else if (warp < WEIGHT_WARP) {
            // ---------------- MMA issuers ----------------
            // Issuer t owns tile t: its accumulator, the items (t, g) and their slots. All four wait for every
            // weight block and release it, also one with nothing to do for the stage: each of its waits and
            // arrivals must count for this use of the weight slot, not for an earlier one (a slot refilled while
            // an issuer has not yet tested its previous use would leave that issuer waiting on the wrong phase).
            // The whole warp walks the stages together: the schedule of the group is worked out once, lane g for
            // stage g (which weight slot and phase, whether tile t takes part, which A slot its item sits in), and
            // handed round with a shuffle, so that the serial part is only waits, the tensor-core instructions of
            // one elected lane (always the same one: commits count the instructions of their own thread) and
            // arrivals.
            if (any) {
                const int t = warp - EPI_WARPS;
                uint32_t info = 0;
                {
                    const uint32_t bits = lane < nstages ? active_tiles<KG>(m, lane) : 0u;
                    int blocks_before = 0;
                    const int items_before = items_before_stage(bits, lane, &blocks_before);
                    const uint32_t pos = a_it + (uint32_t)items_before + (uint32_t)__popc(bits & ((1u << t) - 1u));
                    const uint32_t my_b = b_it + (uint32_t)blocks_before;
                    info = (bits ? 1u : 0u) | (((bits >> t) & 1u) << 1) | ((my_b % B_STAGES) << 2) |
                           (((my_b / B_STAGES) & 1u) << 4) | ((pos % NSLOT) << 5) | (pos << 9);
                }
                // the epilogue must have read this set's previous contents (two groups back)
                bool ok = mbar_wait<false, true>(smem_u32(&ctl->acc_empty[set]), set_phase ^ 1u, abort_flag,
                                                 4 | (int)(acc_it << 4));
                if (ok) tc_fence_after();
                const uint32_t d_tmem = tmem + set * SET_COLS + t * COUT;
                bool started = false;
                for (int g = 0; g < nstages && ok; ++g) {
                    const uint32_t inf = __shfl_sync(0xFFFFFFFFu, info, g);
                    if (!(inf & 1u)) continue;
                    const uint32_t sb = (inf >> 2) & 3u;
                    ok = mbar_wait<false, true>(smem_u32(&ctl->b_full[sb]), (inf >> 4) & 1u, abort_flag,
                                                5 | (int)((b_it + g) << 4));
                    if (!ok) break;
                    if (inf & 2u) {
                        const uint32_t sa = (inf >> 5) & 15u;
                        ok = mbar_wait<false, true>(smem_u32(&ctl->a_full[t][sa]), (full_phase >> sa) & 1u, abort_flag,
                                                    6 | (int)((inf >> 9) << 4));
                        full_phase ^= 1u << sa;   // this issuer's next use of the slot is the next phase
                        if (!ok) break;
                        if (leader) {
                            fence_proxy_async();   // the gathered rows were written through the generic proxy
                            tc_fence_after();
                            const uint64_t adesc = umma_desc(smem_u32(sA + sa * A_BYTES));
                            const uint64_t bdesc = umma_desc(smem_u32(sB + sb * B_BYTES));
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma_f16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, IDESC, (started || kk > 0) ? 1u : 0u);
                            umma_commit(smem_u32(&ctl->a_empty[sa]));   // frees the A slot once these MMAs have read it
                            umma_commit(smem_u32(&ctl->b_empty[sb]));   // and this issuer's hold on the weight block
                        }
                        started = true;
                    } else if (leader) {
                        mbar_arrive(smem_u32(&ctl->b_empty[sb]));   // nothing to read from this weight block
                    }
                }
                if (ok && leader) {
                    if (started) umma_commit(smem_u32(&ctl->acc_full[set]));
                    else mbar_arrive(smem_u32(&ctl->acc_full[set]));
                }
            }
            __syncwarp();
        } else if (warp == INDEX_WARP) {
            // ---------------- neighbour-index loader ----------------
            // Copies, for every item in consumption order, the KG x 128 neighbour indices into the next block of
            // the index ring, two to three slot cycles ahead of the gather warp that will use them. The map is
            // tile-major and spaces a tile's offsets like the index block does, so an item is one bulk copy that
            // reports to the block's barrier by byte count; the lanes of the warp work on IDX_BATCH consecutive
            // items at once (one dependent chain of wait, expect and copy per lane instead of one per item). The
            // gather warps ignore the indices of rows past the frame's row count (stale) and of offsets past kvol
            // (not loaded).
            {
                uint8_t* list = ctl->idx_list;
                {
                    const uint32_t bits = lane < nstages ? active_tiles<KG>(m, lane) : 0u;
                    int at = items_before_stage(bits, lane);
#pragma unroll
                    for (int tt = 0; tt < TILES; ++tt)
                        if ((bits >> tt) & 1u) list[at++] = (uint8_t)((lane << 2) | tt);
                    __syncwarp();
                }
                // The lanes step through the batches together: an item's wait tests the parity of the previous use
                // of its block, which is only meaningful once the lane that handled that use (a lane of an earlier
                // batch) has passed its own wait. A lane running batches ahead of the others would break that.
                bool live = true;
                for (int base = 0; base < n_a; base += IDX_BATCH) {
                    const int e = base + lane;
                    if (live && lane < IDX_BATCH && e < n_a) {
                        const uint32_t q = a_it + (uint32_t)e;
                        const uint32_t j = q % NIDX;
                        const int code = list[e];
                        const int g = code >> 2, t = code & 3;
                        live = mbar_wait(smem_u32(&ctl->i_empty[j]), ((q / NIDX) & 1u) ^ 1u, abort_flag, 7 | (int)(q << 4));
                        if (live) {
                            // the map is tile-major with the block's own spacing between offsets: the stage's
                            // offsets of this tile are one contiguous run
                            int nk = kvol - g * KG;
                            nk = nk > KG ? KG : nk;
                            const uint32_t bar = smem_u32(&ctl->i_full[j]);
                            ctl->idx_uses[j] = q / NIDX + 1u;
                            mbar_arrive_expect_tx(bar, (uint32_t)(nk * TAP_WORDS * 4));
                            bulk_load(smem_u32(&s_idx[j * IDX_WORDS]),
                                      nbr + nbr_index(kvol, max_voxels, b, g * KG, row0 + t * TILE_M),
                                      (uint32_t)(nk * TAP_WORDS * 4), bar);
                        }
                    }
                    live = __all_sync(0xFFFFFFFFu, live);   // also the batch boundary: no lane starts the next batch early
                    if (!live) break;
                }
            }
        } else {
            // ---------------- weight streamer ----------------
            if (lane == 0 && !withhold_weights) {
                uint32_t my_b = b_it;
                for (int g = 0; g < nstages; ++g) {
                    if (!active_tiles<KG>(m, g)) continue;
                    const uint32_t sb = my_b % B_STAGES;
                    if (!mbar_wait(smem_u32(&ctl->b_empty[sb]), ((my_b / B_STAGES) & 1u) ^ 1u, abort_flag,
                                   8 | (int)(my_b << 4)))
                        break;
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
        if (any) ++acc_it;
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // An aborting CTA must not return while its own copies are still writing shared memory or its MMAs tensor
        // memory: the gather and index warps wait for their cp.async copies, the issuers commit to a barrier that
        // warp 4 waits on (bounded) before it frees the tensor memory, the weight streamer waits (bounded) for
        // its last bulk copies.
        if (warp >= FIRST_GATHER_WARP || warp == INDEX_WARP) asm volatile("cp.async.wait_all;" ::: "memory");
        if (warp >= EPI_WARPS && warp < WEIGHT_WARP && leader) umma_commit(smem_u32(&ctl->mma_drain));
        if (warp == INDEX_WARP) {
            for (int j = lane; j < NIDX; j += 32) {
                const uint32_t uses = ctl->idx_uses[j];
                if (!uses) continue;
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&ctl->i_full[j]), (uses - 1u) & 1u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
            }
        }
        if (warp == WEIGHT_WARP && lane == 0) {
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
    if (warp == EPI_WARPS) {
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
    const int smem = umma_smem_bytes<CIN, COUT>();
    static_assert(umma_smem_bytes<CIN, COUT>() <= 227 * 1024, "ring does not fit the shared memory of one SM");
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
    if (!c.scale_host || !c.shift_host) return SESSD_ERR_PARAM;
    EpiConst epi;
    memcpy(epi.scale, c.scale_host, sizeof epi.scale);
    memcpy(epi.shift, c.shift_host, sizeof epi.shift);
    SESSD_LAUNCH_NAMED(name.c_str(), (conv_umma_kernel<CIN, COUT>), persistent_grid(1), Ring<CIN>::THREADS, smem, stream,
                       static_cast<const __half*>(c.in), static_cast<__half*>(c.out), c.nbr, c.tile_mask, c.out_num,
                       static_cast<const uint8_t*>(c.umma_weights), epi, c.relu, c.batch, c.max_voxels,
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
