// Steps 2+3 of the AMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The gather  acc[m][n] = sum_cb LUT[cb][idx[m][cb]][n]  is the contraction
//     acc[M x N] = OneHot[M x (CB*CT)] * LUT[(CB*CT) x N]
// with OneHot[m][cb*CT + c] = (idx[m][cb] == c).  All operands are small integers and the
// accumulator is int32, so tcgen05.mma kind::i8 gives exactly the sums the reference's DPU
// kernel produces (inference-engine/src/dpu/pim_lut_kernel.c:159-175; canonical statement
// inference-engine/test/test_amm.cpp:164-175), in a different but irrelevant order.
// It does CT times more multiply-adds than the gather, on a pipe that is far more than
// CT times faster.  The dequantisation (inference-engine/src/host/pim_lut_host.cpp:201)
// is fused into the epilogue.
//
// Persistent kernel: one CTA per SM walks a list of work items, an item being one
// 128-token x N_TILE-column output tile, or one slice of its contraction axis when
// split > 1 (each slice then writes its int32 partial tile to scratch in L2 with plain
// stores, and the CTAs holding a tile's slices sum it together and dequantise).
// The accumulator is double-buffered in TMEM so the epilogue of one item overlaps the
// main loop of the next.  Operands move through two rings of 128-byte slabs of the contraction
// axis: LUT slabs in shared memory (as many as fit), one-hot slabs in tensor memory or shared
// memory (what the accumulators, resp. the LUT ring, leave).
//
//   warp 0        TMA producer: B slabs = LUT^T[n0:n0+N_TILE][k:k+128] (K-major, 128-byte
//                 swizzle) from the load-time transposed copy of the LUT
//   warps 1-2     issue tcgen05.mma, 4 per slab, slab x by warp 1 + x % 2 (one elected lane);
//                 warp 1 also owns TMEM (alloc/dealloc)
//   warps 3-18    build the one-hot A slab straight from the uint8 indices (it never exists in
//                 HBM): four groups of four warps, group k taking every fourth slab, one tile
//                 row per thread, the row's eight 16-byte chunks read from a one-hot table in
//                 shared memory.  Four groups because a slab is a chain of latencies (index
//                 load, wait, fence, arrive): they have to overlap across slabs.
//   warps 19-22   epilogue: TMEM -> registers -> shared-memory transpose -> dequantise ->
//                 row-contiguous 16-byte global stores (each warp owns one 32-lane quadrant);
//                 clears the accumulator behind itself
//
// HBM traffic: M*CB (indices) + CB*CT*N (LUT^T, once if L2-resident across M tiles)
//              + 4*N (bias) + 4*M*N (output).
#include "kernels.h"
#include "ptx.cuh"
#include "epilogue.cuh"

namespace lutamm {

namespace {

constexpr uint32_t kMTile = 128;
constexpr uint32_t kSlabK = 128;               // bytes of K per pipeline stage = one swizzle row
constexpr uint32_t kABytes = kMTile * kSlabK;  // 16 KiB
constexpr uint32_t kMaxAgenGroups = 4;  // each group: 4 warps = 128 rows (more groups measured slower)
constexpr uint32_t kEpiWarps = 4;
constexpr uint32_t kEpiThreads = kEpiWarps * 32;
constexpr uint32_t kMmaWarps = 2;      // MMA-issuing warps: slab x of the CTA's sequence is issued by warp x % 2
constexpr uint32_t kFirstAgenWarp = 1 + kMmaWarps;
constexpr uint32_t kMaxThreads = (kFirstAgenWarp + 4 * kMaxAgenGroups + kEpiWarps) * 32;  // 736
constexpr uint32_t kMaxASlots = 8;    // one-hot slabs in flight (tensor memory: 32 columns each)
constexpr uint32_t kMaxBSlots = 16;   // LUT slabs in flight (shared memory)
constexpr uint32_t kNumBarriers = 2 * kMaxASlots + 2 * kMaxBSlots + 4;
constexpr uint32_t kStageWarpBytes = 32 * 128;           // epilogue transpose buffer per warp
constexpr uint32_t kBiasWarpBytes = 256 * 4;             // a tile's bias values, one copy per epilogue warp (store-by-copy-engine epilogue)
// One-hot table: row e (0..15) holds the 16 bytes "byte e = 1", row 16 holds zeros; a row is 128
// bytes = eight copies, and lane l reads copy l % 8, so a 16-byte load is free of bank conflicts
// whatever indices the lanes of a warp hold.
constexpr uint32_t kOneHotRows = 17;
constexpr uint32_t kOneHotTabBytes = kOneHotRows * 128;

struct UmmaParams {
    LutArgs a;
    uint32_t slabs_total;    // ceil(CB*CT / 128)
    uint32_t slabs_per_item; // ceil(slabs_total / split)
    uint32_t split;
    uint32_t a_slots;        // ring of one-hot slabs (tensor memory or shared memory)
    uint32_t a_slots_magic;  // ceil(2^32 / a_slots): slab x lives in slot x % a_slots, found without a division
    uint32_t b_slots;        // ring of LUT slabs (shared memory), at least a_slots
    uint32_t tiles_m, tiles_n;
    uint32_t log2_ct;
    uint32_t groups;         // A-builder groups (1..4); a_slots % (groups * slabs per turn) == 0
    uint32_t early_trigger;  // 1: let the next kernel of the stream start once this CTA's main loops are done
    int32_t* acc_scratch;    // [split][M][N] int32 partial sums (split > 1); needs no initialisation
    uint32_t* tile_counters;
    uint32_t* dev_err;
};

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t n) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}
// 32-bit left shift with PTX semantics: a shift amount of 32 or more gives 0 (shl.b32 clamps).
__device__ __forceinline__ uint32_t shl32_clamped(uint32_t v, uint32_t n) {
    uint32_t r;
    asm("shl.b32 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(n));
    return r;
}
// 16 bytes with byte `i` set to 1, given n = 8*i; any n >= 128 gives zeros.  Word w of the result
// is 1 << (n - 32*w) under the clamping shift: for n below the word the subtraction wraps to a
// huge amount, for n above it the amount is 32 or more, and both give zero.
__device__ __forceinline__ uint4 onehot16_bits(uint32_t n) {
    return make_uint4(shl32_clamped(1u, n), shl32_clamped(1u, n - 32u), shl32_clamped(1u, n - 64u),
                      shl32_clamped(1u, n - 96u));
}
__device__ __forceinline__ uint4 onehot16(uint32_t i) { return onehot16_bits(i < 16u ? i * 8u : 128u); }

// x / d for x * d < 2^32, given magic = ceil(2^32 / d): one multiply-high.
__device__ __forceinline__ uint32_t div_magic(uint32_t x, uint32_t magic) { return __umulhi(x, magic); }

struct Item {
    uint32_t m0, n0, slab_begin, nslab, tile, z;
};
__device__ __forceinline__ uint32_t rsw_of(uint32_t row) { return row & 7u; }
__device__ __forceinline__ Item decode_item(const UmmaParams& p, uint32_t item, uint32_t n_tile) {
    Item it;
    const uint32_t z = item % p.split, tile = item / p.split;
    it.tile = tile;
    it.z = z;
    it.m0 = (tile % p.tiles_m) * kMTile;
    it.n0 = (tile / p.tiles_m) * n_tile;
    it.slab_begin = z * p.slabs_per_item;
    const uint32_t end = min(p.slabs_total, it.slab_begin + p.slabs_per_item);
    it.nslab = end > it.slab_begin ? end - it.slab_begin : 0u;
    return it;
}

template <uint32_t N_TILE, bool A_TMEM, uint32_t SPS, bool PEER = false, bool EPI_TMA = false>
__global__ void __launch_bounds__(kMaxThreads, 1)
lut_onehot_umma_kernel(const __grid_constant__ CUtensorMap lut_t_map, const UmmaParams p, const __grid_constant__ CUtensorMap out_map) {
    constexpr uint32_t kBBytes = N_TILE * kSlabK;
    constexpr uint32_t kIdesc = umma_idesc_i8(kMTile, N_TILE, /*a_signed=*/1, /*b_signed=*/1);
    // Tensor memory: two accumulators of N_TILE columns; with A_TMEM also the ring of one-hot
    // A slabs (32 columns = 128 bytes of K per row) behind them.
    constexpr uint32_t kTmemCols = A_TMEM ? 512u : (2 * N_TILE <= 32 ? 32u : 2 * N_TILE <= 64 ? 64u : 2 * N_TILE <= 128 ? 128u : 2 * N_TILE <= 256 ? 256u : 512u);
    constexpr uint32_t kATmemBase = 2 * N_TILE;
    constexpr uint32_t kASlotBytes = A_TMEM ? 0u : kABytes;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // Two rings, one slab (128 bytes of the contraction axis) per slot.  The LUT ring is as deep as
    // shared memory allows: a TMA tile takes on the order of a microsecond to arrive, several slab
    // times, and it is the number of tiles in flight that hides it.  The one-hot ring is bounded by
    // tensor memory (what the two accumulators leave) or, in shared memory, by what the LUT ring leaves.
    const uint32_t SA = p.a_slots, SB = p.b_slots;
    unsigned char* s_a = smem;                                   // [SA][16 KiB], 1024-aligned (A in shared memory only)
    unsigned char* s_b = s_a + (size_t)SA * kASlotBytes;         // [SB][N_TILE*128], 1024-aligned
    unsigned char* s_stage = s_b + (size_t)SB * kBBytes;         // [4][32][128] epilogue transpose
    unsigned char* s_tab = s_stage + kEpiWarps * kStageWarpBytes;  // one-hot table, 128-byte aligned
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_tab + kOneHotTabBytes);
    uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_bar + kNumBarriers);  // tmem base, abort, last
    float* s_bias = reinterpret_cast<float*>(s_misc + 4);                  // [4][256] (EPI_TMA only)
    volatile uint32_t* s_abort = s_misc + 1;

    const uint32_t a_full0 = smem_u32(s_bar), a_empty0 = a_full0 + 8 * kMaxASlots, b_full0 = a_empty0 + 8 * kMaxASlots,
                   b_empty0 = b_full0 + 8 * kMaxBSlots, acc_full0 = b_empty0 + 8 * kMaxBSlots, acc_empty0 = acc_full0 + 16;

    const LutArgs& a = p.a;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_items = p.tiles_m * p.tiles_n * p.split;
    const uint32_t kAgenGroups = p.groups;
    const uint32_t kFirstEpiWarp = kFirstAgenWarp + 4 * kAgenGroups;

    // Set-up, spread over the CTA so that nothing waits for one thread: a barrier per thread of warps 2 and 3
    // (one thread initialising all 52 took 1 400 cycles), the one-hot table by warps 4 to 8, and warp 1
    // allocates tensor memory meanwhile; with one tile per CTA this prologue is on the critical path, since the
    // CTA only becomes resident when the search kernel before it leaves the SM.
    if (threadIdx.x == 0) {
        s_misc[1] = 0; s_misc[2] = 0;   // [0] is written by tcgen05.alloc
        tma_prefetch_desc(&lut_t_map);
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + kNumBarriers) {
        const uint32_t b = threadIdx.x - 64;
        // a_full: the four builder warps of the group that owns the slab; a_empty, b_empty: one tcgen05.commit;
        // b_full: the producer's arrive.expect_tx (the TMA completes the bytes); acc_full: one commit per
        // issuing warp; acc_empty: the epilogue warps
        const uint32_t count = b < kMaxASlots ? 4u : b < 2 * kMaxASlots + 2 * kMaxBSlots ? 1u : b < 2 * kMaxASlots + 2 * kMaxBSlots + 2 ? kMmaWarps : kEpiWarps;
        mbar_init(a_full0 + 8 * b, count);
        fence_barrier_init();
    }
    if (threadIdx.x >= 128 && threadIdx.x < 128 + kOneHotRows * 8) {
        const uint32_t e = (threadIdx.x - 128) >> 3, copy = (threadIdx.x - 128) & 7u;
        *reinterpret_cast<uint4*>(s_tab + e * 128 + copy * 16) = onehot16(e);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(s_misc), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_misc);
    // Every MMA accumulates (two warps issue them, in no fixed order), so the accumulators start at
    // zero: the epilogue warps clear both here and clear each again after reading it.
    if (warp >= kFirstEpiWarp) {
        const uint32_t zero[32] = {};
        for (uint32_t c = 0; c < 2 * N_TILE / 32; ++c)
            tmem_st_32x32b_x32(tmem_base + (((warp & 3u) * 32u) << 16) + c * 32u, zero);
        tmem_st_wait();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    if (warp == 0) {
        // ---------------- TMA producer (the LUT never depends on the preceding kernel)
        if (lane == 0) {
            uint32_t j = 0, ph = 0;  // LUT slot and the phase bit of its current use
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item it = decode_item(p, item, N_TILE);
                for (uint32_t i = 0; i < it.nslab; ++i) {
                    ok = mbar_wait<32>(b_empty0 + 8 * j, ph ^ 1, s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(b_full0 + 8 * j, kBBytes);
                    tma_load_2d(smem_u32(s_b + (size_t)j * kBBytes), &lut_t_map, b_full0 + 8 * j,
                                (int32_t)((it.slab_begin + i) * kSlabK), (int32_t)it.n0);
                    if (++j == SB) { j = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();
        if (p.early_trigger) pdl_launch_dependents();
    } else if (warp < kFirstAgenWarp) {
        // ---------------- MMA issuers: two warps, slab x of the CTA's sequence goes to warp x % 2.
        // A slab's turn (barrier probes, fence, election, four tcgen05.mma of 32 bytes of K each, one
        // commit per ring) costs the issuing warp about 600 cycles, more than the four MMAs take to
        // execute; two warps taking turns keep the tensor pipe fed.  All MMAs accumulate into an
        // accumulator the epilogue left at zero, integer addition commutes, so the order in which
        // the two warps' instructions reach the pipe does not matter.  Each warp walks its loop
        // converged (waits and descriptor arithmetic stay warp-uniform; a lone lane running the
        // loop measured 20 % slower), one elected lane issues.
        {
            const uint32_t me = warp - 1;
            const uint32_t sa_magic = p.a_slots_magic;
            auto a_slot = [&](uint32_t x, uint32_t& k, uint32_t& pa) { const uint32_t q = div_magic(x, sa_magic); k = x - q * SA; pa = q & 1u; };
            uint32_t j = me % SB, pb = 0, t = 0, x0 = 0;  // LUT slot / phase of this warp's next slab; slabs before the item
            bool ok = true;
            const uint32_t b_lo0 = (uint32_t)umma_desc_k_sw128(smem_u32(s_b));
            const uint32_t a_lo0 = (uint32_t)umma_desc_k_sw128(smem_u32(s_a));
            const uint32_t desc_hi = (uint32_t)(umma_desc_k_sw128(0) >> 32);
            // Whether a slab's two slots are full is asked one turn ahead: a barrier query is a round
            // trip of the order of a hundred cycles.
            uint32_t k, pa;
            a_slot(me, k, pa);
            bool ready = mbar_test2(b_full0 + 8 * j, pb, a_full0 + 8 * k, pa);
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++t) {
                const Item it = decode_item(p, item, N_TILE);
                const uint32_t ab = t & 1, aph = (t >> 1) & 1;
                ok = mbar_wait(acc_empty0 + 8 * ab, aph ^ 1, s_abort);  // epilogue drained and cleared this buffer
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + ab * N_TILE;
                for (uint32_t i = (x0 + me) & 1u; i < it.nslab; i += 2) {
                    const uint32_t x = x0 + i;
                    a_slot(x, k, pa);
                    if (!ready) {
                        ok = mbar_wait(b_full0 + 8 * j, pb, s_abort) && mbar_wait(a_full0 + 8 * k, pa, s_abort);
                        if (!ok) break;
                    }
                    uint32_t j2 = j + 2, pb2 = pb;
                    if (j2 >= SB) { j2 -= SB; pb2 ^= 1; }
                    uint32_t k2, pa2;
                    a_slot(x + 2, k2, pa2);
                    const bool next_ready = mbar_test2(b_full0 + 8 * j2, pb2, a_full0 + 8 * k2, pa2);
                    tc_fence_after_sync();
                    if (elect_one()) {
                        // descriptors differ from slot 0's only in the 16-byte-unit address field
                        const uint32_t b_lo = b_lo0 + j * (kBBytes >> 4);
                        if constexpr (A_TMEM) {
                            const uint32_t ta = tmem_base + kATmemBase + k * 32;
#pragma unroll
                            for (uint32_t kk = 0; kk < kSlabK / 32; ++kk)  // 32 bytes of K = 8 TMEM columns of A
                                umma_i8_ts(d_tmem, ta + 8 * kk, ((uint64_t)desc_hi << 32) | (b_lo + 2 * kk), kIdesc, 1u);
                        } else {
                            const uint32_t a_lo = a_lo0 + k * (kABytes >> 4);
#pragma unroll
                            for (uint32_t kk = 0; kk < kSlabK / 32; ++kk)  // 32 bytes of K per instruction
                                umma_i8(d_tmem, ((uint64_t)desc_hi << 32) | (a_lo + 2 * kk),
                                        ((uint64_t)desc_hi << 32) | (b_lo + 2 * kk), kIdesc, 1u);
                        }
                        umma_commit(a_empty0 + 8 * k);  // each slot is free once these MMAs have read it
                        umma_commit(b_empty0 + 8 * j);
                    }
                    __syncwarp();
                    j = j2; pb = pb2;
                    ready = next_ready;
                }
                x0 += it.nslab;
                if (ok && elect_one()) umma_commit(acc_full0 + 8 * ab);  // this warp's share of the item is issued
                __syncwarp();
            }
        }
        __syncwarp();
        if (p.early_trigger) pdl_launch_dependents();
    } else if (warp < kFirstEpiWarp) {
        // ---------------- one-hot A builders: groups of 4 warps; group k owns every
        // kAgenGroups-th slab of the CTA's slab sequence, one tile row per thread, so the
        // fixed latencies of a slab (index load, wait, fence, arrive) overlap across groups
        // instead of adding up.
        // The indices come from the kernel launched just before; ld.global.cg reads them from
        // L2, which matters because under programmatic dependent launch this CTA may have
        // started, on an SM with older lines in L1, before that kernel finished.
        pdl_wait_prior_grid();
        const uint32_t grp = (warp - kFirstAgenWarp) >> 2;
        const uint32_t r = (warp & 3u) * 32 + lane;  // tile row == TMEM lane
        const uint32_t sw = r & 7u;
        const uint32_t CT = a.CT, lg = p.log2_ct;
        const unsigned char* tab_lane = s_tab + (lane & 7u) * 16;
        // bytes of index one slab needs per row: 128 / CT codebooks (at least one byte)
        auto load_raw = [&](const uint8_t* row, uint32_t slab) -> uint4 {
            const uint8_t* q = row + ((slab * kSlabK) >> lg);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (lg == 4) { const uint2 t = __ldcg(reinterpret_cast<const uint2*>(q)); v.x = t.x; v.y = t.y; }
            else if (lg == 3) v = __ldcg(reinterpret_cast<const uint4*>(q));
            else if (lg == 5) v.x = __ldcg(reinterpret_cast<const uint32_t*>(q));
            else if (lg == 6) v.x = __ldcg(reinterpret_cast<const uint16_t*>(q));
            else v.x = __ldcg(q);
            return v;
        };
        // A group takes SPS consecutive slabs per turn: the fixed cost of a turn - the fences, the
        // arrival, the loop itself, a chain of latencies of many hundred cycles for a lone warp - is
        // then paid once per batch.  Batch q of the CTA's sequence goes to group q % groups; slab x of
        // the sequence uses one-hot slot x % SA.
        constexpr uint32_t kBatch = SPS;
        // Index bytes are fetched kPrefetch turns ahead: with the LUT tiles streaming through the same
        // L2 a load takes a good part of a turn.
        constexpr uint32_t kPrefetch = 2;
        const uint32_t sa_magic = p.a_slots_magic;
        uint32_t ga = 0, qb = 0;  // slabs and batches of the CTA before the current item
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const Item it = decode_item(p, item, N_TILE);
            const uint8_t* grow = a.idx + (size_t)min(it.m0 + r, a.M - 1) * a.CB;  // rows past M: masked in the epilogue
            uint32_t i = kBatch * ((grp + kAgenGroups - (qb % kAgenGroups)) % kAgenGroups);  // first slab of the turn
            const uint32_t stride = kBatch * kAgenGroups;
            uint4 raw_q[kPrefetch][kBatch];
#pragma unroll
            for (uint32_t k = 0; k < kPrefetch; ++k)
#pragma unroll
                for (uint32_t b = 0; b < kBatch; ++b) {
                    raw_q[k][b] = make_uint4(0, 0, 0, 0);
                    if (i + k * stride + b < it.nslab) raw_q[k][b] = load_raw(grow, it.slab_begin + i + k * stride + b);
                }
            for (; i < it.nslab && ok; i += stride) {
                uint4 raw[kBatch];
#pragma unroll
                for (uint32_t b = 0; b < kBatch; ++b) {
                    raw[b] = raw_q[0][b];
#pragma unroll
                    for (uint32_t k = 0; k + 1 < kPrefetch; ++k) raw_q[k][b] = raw_q[k + 1][b];
                    if (i + kPrefetch * stride + b < it.nslab)
                        raw_q[kPrefetch - 1][b] = load_raw(grow, it.slab_begin + i + kPrefetch * stride + b);
                }
#pragma unroll
                for (uint32_t b = 0; b < kBatch; ++b) {
                    if (i + b >= it.nslab) continue;  // an odd last batch
                    const uint32_t slab = it.slab_begin + i + b;
                    const uint32_t x = ga + i + b, xq = div_magic(x, sa_magic), k = x - xq * SA, pa = xq & 1u;
                    // Row of the one-hot table per 16-byte chunk, then one conflict-free 16-byte load each.
                    // An index that is out of range for its chunk selects the all-zero row (the indices
                    // may come from a caller, not only from the search kernel).
                    uint4 chunk[8];
                    if (lg == 4) {  // one codebook == one 16-byte chunk
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) {
                            const uint32_t ix = ((j < 4 ? raw[b].x : raw[b].y) >> (8 * (j & 3))) & 0xFFu;
                            chunk[j] = *reinterpret_cast<const uint4*>(tab_lane + min(ix, 16u) * 128);
                        }
                    } else if (lg == 3) {  // two codebooks per chunk: low eight bytes, high eight bytes
                        const uint32_t w[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) {
                            const uint32_t two = (w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
                            const uint32_t i0 = two & 0xFFu, i1 = two >> 8;
                            const uint4 lo = *reinterpret_cast<const uint4*>(tab_lane + (i0 < 8u ? i0 : 16u) * 128);
                            const uint4 hi = *reinterpret_cast<const uint4*>(tab_lane + (i1 < 8u ? i1 + 8u : 16u) * 128);
                            chunk[j] = make_uint4(lo.x | hi.x, lo.y | hi.y, lo.z | hi.z, lo.w | hi.w);
                        }
                    } else {  // a codebook spans CT/16 chunks
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) {
                            const uint32_t k0 = slab * kSlabK + 16 * j;
                            const uint32_t ix = (raw[b].x >> (8 * (j >> (lg - 4)))) & 0xFFu;  // CT >= 128: always byte 0
                            const uint32_t sub = (k0 & (CT - 1)) >> 4;
                            chunk[j] = *reinterpret_cast<const uint4*>(tab_lane + ((ix >> 4) == sub ? (ix & 15u) : 16u) * 128);
                        }
                    }
                    // The row is in registers before the slot is waited for: what follows the wait is on
                    // the slot's turn-around path.  The whole warp polls (one broadcast access), so it
                    // stays converged.
                    ok = ok && mbar_wait(a_empty0 + 8 * k, pa ^ 1, s_abort);
                    if (!ok) continue;
                    if constexpr (A_TMEM) {
                        tc_fence_after_sync();
                        // the row goes to this warp's lane quadrant of tensor memory, K bytes in column order
                        uint32_t w[32];
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) {
                            w[4 * j + 0] = chunk[j].x; w[4 * j + 1] = chunk[j].y; w[4 * j + 2] = chunk[j].z; w[4 * j + 3] = chunk[j].w;
                        }
                        tmem_st_32x32b_x32(tmem_base + (((warp & 3u) * 32u) << 16) + kATmemBase + k * 32, w);
                    } else {
                        unsigned char* row_ptr = s_a + (size_t)k * kABytes + r * kSlabK;
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j)  // 128-byte swizzle: 16-byte chunk j of row r lands at j ^ (r & 7)
                            *reinterpret_cast<uint4*>(row_ptr + ((j ^ sw) << 4)) = chunk[j];
                    }
                }
                if constexpr (A_TMEM) {
                    tmem_st_wait();
                    tc_fence_before_sync();
                } else {
                    fence_proxy_async_smem();
                }
                __syncwarp();
                if (lane == 0 && ok) {
#pragma unroll
                    for (uint32_t b = 0; b < kBatch; ++b)
                        if (i + b < it.nslab) {
                            const uint32_t x = ga + i + b;
                            mbar_arrive(a_full0 + 8 * (x - div_magic(x, sa_magic) * SA));
                        }
                }
            }
            ga += it.nslab;
            qb += (it.nslab + kBatch - 1) / kBatch;
        }
        if (p.early_trigger) pdl_launch_dependents();
    } else {
        // ---------------- epilogue: four warps, each on the TMEM lane quadrant (warp % 4) it may read
        pdl_wait_prior_grid();
        const uint32_t quad = warp & 3u;
        const uint32_t et = threadIdx.x - kFirstEpiWarp * 32;
        const float lbcb = lut_bias_times_cb(a.lut_bias, a.CB);
        unsigned char* stg = s_stage + (warp - kFirstEpiWarp) * kStageWarpBytes;
        if constexpr (EPI_TMA) {
            // The tile leaves through the copy engine: each thread dequantises the 32 columns of its own row in
            // the layout tcgen05.ld delivers, writes them as eight 16-byte shared-memory stores (128-byte swizzle,
            // conflict free) and one lane hands the 32 x 32 block to a tiled store, which also clips rows past M
            // and columns past N.  A third of the instructions of the transposing path below, and no load/store-unit
            // traffic for the global stores: what the epilogue issues is taken from the builders' latency chain.
            // (Launches with split tiles, tiled output, an int32 copy or peer stores use the path below.)
            float* bw = s_bias + (warp - kFirstEpiWarp) * (kBiasWarpBytes / 4);
            if (lane == 0) tma_prefetch_desc(&out_map);
            uint32_t t = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++t) {
                const Item it = decode_item(p, item, N_TILE);
                const uint32_t ab = t & 1, aph = (t >> 1) & 1;
                if (p.early_trigger && item + gridDim.x >= n_items) pdl_launch_dependents();
                __syncwarp();  // the previous item's reads of bw are done
#pragma unroll
                for (uint32_t c = 0; c < N_TILE / 32; ++c) {
                    const uint32_t n = it.n0 + c * 32 + lane;
                    bw[c * 32 + lane] = n < a.N ? __ldg(a.bias + n) : 0.f;
                }
                uint32_t w_ok = 1;
                if (lane == 0) w_ok = (ok && mbar_wait<256>(acc_full0 + 8 * ab, aph, s_abort)) ? 1u : 0u;
                ok = __shfl_sync(0xffffffffu, w_ok, 0) != 0;
                if (!ok) continue;
                tc_fence_after_sync();
                for (uint32_t c = 0; c < N_TILE / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + ((quad * 32u) << 16) + ab * N_TILE + c * 32u, v);
                    tmem_ld_wait();
                    {   // leave the columns at zero for the next item's accumulating MMAs
                        const uint32_t zero[32] = {};
                        tmem_st_32x32b_x32(tmem_base + ((quad * 32u) << 16) + ab * N_TILE + c * 32u, zero);
                    }
                    if (c == N_TILE / 32 - 1) {  // accumulator fully read and cleared: hand the buffer back
                        tmem_st_wait();
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty0 + 8 * ab);
                    }
                    if (it.n0 + c * 32 >= a.N || it.m0 + quad * 32 >= a.M) continue;  // a block wholly past N or M (warp-uniform)
                    // the previous block's copy has read the staging buffer
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bw + c * 32 + 4 * q);
                        float4 o = make_float4(dequant_one((int32_t)v[4 * q], a.scale, lbcb, b4.x), dequant_one((int32_t)v[4 * q + 1], a.scale, lbcb, b4.y),
                                               dequant_one((int32_t)v[4 * q + 2], a.scale, lbcb, b4.z), dequant_one((int32_t)v[4 * q + 3], a.scale, lbcb, b4.w));
                        if (a.act) { o.x = activate_one(o.x, a.act); o.y = activate_one(o.y, a.act); o.z = activate_one(o.z, a.act); o.w = activate_one(o.w, a.act); }
                        *reinterpret_cast<float4*>(stg + lane * 128 + ((q ^ rsw_of(lane)) << 4)) = o;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&out_map, smem_u32(stg), (int32_t)(it.n0 + c * 32), (int32_t)(it.m0 + quad * 32));
                        tma_store_commit();
                    }
                }
            }
            if (lane == 0) tma_store_wait_all();  // shared memory and the output are settled before the CTA leaves
            __syncwarp();
            tc_fence_before_sync();
        } else {
        const uint32_t rsw = lane & 7u;
        const uint32_t ch = lane & 7u, rsub = lane >> 3;  // store phase: 16-byte column group, row within a pass
        uint32_t t = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++t) {
            const Item it = decode_item(p, item, N_TILE);
            const uint32_t ab = t & 1, aph = (t >> 1) & 1;
            if (p.early_trigger && item + gridDim.x >= n_items) pdl_launch_dependents();
            // The bias values are fetched one chunk ahead, the first before the accumulator is
            // waited for: a miss to DRAM would otherwise sit on the critical path of every chunk.
            auto load_bias = [&](uint32_t c) -> float4 {
                const uint32_t n = it.n0 + c * 32 + ch * 4;
                return n < a.N ? __ldg(reinterpret_cast<const float4*>(a.bias + n)) : make_float4(0.f, 0.f, 0.f, 0.f);
            };
            float4 b_next = load_bias(0);
            uint32_t w_ok = 1;
            if (lane == 0) w_ok = (ok && mbar_wait<256>(acc_full0 + 8 * ab, aph, s_abort)) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, w_ok, 0) != 0;
            if (ok) {
                tc_fence_after_sync();
                for (uint32_t c = 0; c < N_TILE / 32; ++c) {
                    const float4 b4 = b_next;
                    if (c + 1 < N_TILE / 32) b_next = load_bias(c + 1);
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + ((quad * 32u) << 16) + ab * N_TILE + c * 32u, v);
                    tmem_ld_wait();
                    {   // leave the columns at zero for the next item's accumulating MMAs
                        const uint32_t zero[32] = {};
                        tmem_st_32x32b_x32(tmem_base + ((quad * 32u) << 16) + ab * N_TILE + c * 32u, zero);
                    }
                    if (c == N_TILE / 32 - 1) {  // accumulator fully read and cleared: hand the buffer back
                        tmem_st_wait();
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty0 + 8 * ab);
                    }
                    __syncwarp();
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((q ^ rsw) << 4)) =
                            make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    __syncwarp();
                    const uint32_t n = it.n0 + c * 32 + ch * 4;
                    if (n < a.N) {  // N % 16 == 0: a 4-column group is in or out as a whole
                        // One warp per scheduler is all that runs here, so the eight row passes are
                        // written as straight-line code with their loads, conversions and stores
                        // grouped: a pass-by-pass loop leaves every latency exposed.
                        const uint32_t m_first = it.m0 + quad * 32 + rsub;  // row of pass 0; pass k is 4k rows further
#pragma unroll
                        for (uint32_t half = 0; half < 2; ++half) {  // four passes at a time: registers
                            int4 val[4];
#pragma unroll
                            for (uint32_t k = 0; k < 4; ++k) {
                                const uint32_t rr = (half * 4 + k) * 4 + rsub;
                                val[k] = *reinterpret_cast<const int4*>(stg + rr * 128 + ((ch ^ (rr & 7u)) << 4));
                            }
                            const uint32_t m_half = m_first + half * 16;
                            if (p.split > 1) {  // this slice's partial sums, plain row-contiguous stores
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k)
                                    if (m_half + k * 4 < a.M)
                                        __stcg(reinterpret_cast<int4*>(p.acc_scratch + ((size_t)it.z * a.M + m_half + k * 4) * a.N + n), val[k]);
                                continue;
                            }
                            float4 o[4];
#pragma unroll
                            for (uint32_t k = 0; k < 4; ++k) {
                                o[k].x = dequant_one(val[k].x, a.scale, lbcb, b4.x);
                                o[k].y = dequant_one(val[k].y, a.scale, lbcb, b4.y);
                                o[k].z = dequant_one(val[k].z, a.scale, lbcb, b4.z);
                                o[k].w = dequant_one(val[k].w, a.scale, lbcb, b4.w);
                            }
                            if (a.act) {
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k) {
                                    o[k].x = activate_one(o[k].x, a.act);
                                    o[k].y = activate_one(o[k].y, a.act);
                                    o[k].z = activate_one(o[k].z, a.act);
                                    o[k].w = activate_one(o[k].w, a.act);
                                }
                            }
                            if (!a.layout.tiled) {
                                float* orow = a.out + (size_t)m_half * a.N + n;
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k)
                                    if (m_half + k * 4 < a.M) *reinterpret_cast<float4*>(orow + (size_t)k * 4 * a.N) = o[k];
                                if constexpr (PEER) {  // the same rows into every other GPU's gathered buffer
                                    for (uint32_t g = 0; g < a.n_peers; ++g) {
                                        if (a.peer_out[g] == a.out) continue;
                                        float* prow = a.peer_out[g] + (size_t)m_half * a.N + n;
#pragma unroll
                                        for (uint32_t k = 0; k < 4; ++k)
                                            if (m_half + k * 4 < a.M) *reinterpret_cast<float4*>(prow + (size_t)k * 4 * a.N) = o[k];
                                    }
                                }
                            } else {
                                for (uint32_t k = 0; k < 4; ++k) {
                                    const uint32_t mm = m_half + k * 4;
                                    if (mm >= a.M) continue;
                                    a.out[tiled_out_offset(mm, n + 0, a.layout)] = o[k].x;
                                    a.out[tiled_out_offset(mm, n + 1, a.layout)] = o[k].y;
                                    a.out[tiled_out_offset(mm, n + 2, a.layout)] = o[k].z;
                                    a.out[tiled_out_offset(mm, n + 3, a.layout)] = o[k].w;
                                }
                            }
                            if (a.acc_out) {
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k)
                                    if (m_half + k * 4 < a.M)
                                        *reinterpret_cast<int4*>(a.acc_out + (size_t)(m_half + k * 4) * a.N + n) = val[k];
                            }
                        }
                    }
                }
            }
            if (p.split > 1) {
                // The CTAs that hold the slices of an output tile sum them together: each waits (bounded)
                // until all slices are in the scratch buffer, then sums and dequantises its share of
                // the tile's rows - row pass p of every 32-row quadrant goes to slice p % split.  (One
                // CTA summing the whole tile took longer than the main loop of a short slice.)  The
                // grid never exceeds one CTA per SM and a CTA takes its items in increasing order, so
                // the slices of a tile are in progress or done when one of them waits here.
                // Every epilogue thread runs the barriers, also after a failed wait, so nobody is left
                // behind at one.
                __threadfence();
                named_bar_sync(1, kEpiThreads);
                uint32_t* ctr = p.tile_counters + 2 * it.tile;  // [0] slices arrived, [1] slices done
                if (et == 0) {
                    uint32_t go = 0;
                    if (ok && !*s_abort) {
                        atomicAdd(ctr, 1u);
                        for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
                            if (*reinterpret_cast<volatile uint32_t*>(ctr) >= p.split) { go = 1; break; }
                            if ((spin & 63u) == 63u && *s_abort) break;
                            __nanosleep(64);
                        }
                        if (!go) *s_abort = 1u;
                    }
                    s_misc[2] = go;
                }
                named_bar_sync(1, kEpiThreads);
                if (s_misc[2]) {
                    __threadfence();
                    // All loads of a row first, then the stores: the loop is a chain of L2 round
                    // trips otherwise.
                    constexpr uint32_t kChunks = N_TILE / 32;
                    for (uint32_t pass = it.z; pass < 8; pass += p.split) {
                        const uint32_t mm = it.m0 + quad * 32 + pass * 4 + rsub;
                        if (mm >= a.M) continue;
                        int4 val[kChunks];
#pragma unroll
                        for (uint32_t c = 0; c < kChunks; ++c) val[c] = make_int4(0, 0, 0, 0);
                        for (uint32_t z = 0; z < p.split; ++z) {  // integer sums: the order is immaterial
                            int4 part[kChunks];
#pragma unroll
                            for (uint32_t c = 0; c < kChunks; ++c) {
                                const uint32_t n = it.n0 + c * 32 + ch * 4;
                                part[c] = make_int4(0, 0, 0, 0);
                                if (n < a.N) part[c] = __ldcg(reinterpret_cast<const int4*>(p.acc_scratch + ((size_t)z * a.M + mm) * a.N + n));
                            }
#pragma unroll
                            for (uint32_t c = 0; c < kChunks; ++c) {
                                val[c].x += part[c].x; val[c].y += part[c].y; val[c].z += part[c].z; val[c].w += part[c].w;
                            }
                        }
#pragma unroll
                        for (uint32_t c = 0; c < kChunks; ++c) {
                            const uint32_t n = it.n0 + c * 32 + ch * 4;
                            if (n >= a.N) continue;
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(a.bias + n));
                            float o[4] = {dequant_one(val[c].x, a.scale, lbcb, b4.x), dequant_one(val[c].y, a.scale, lbcb, b4.y),
                                          dequant_one(val[c].z, a.scale, lbcb, b4.z), dequant_one(val[c].w, a.scale, lbcb, b4.w)};
                            if (a.act) {
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k) o[k] = activate_one(o[k], a.act);
                            }
                            if (!a.layout.tiled) {
                                *reinterpret_cast<float4*>(a.out + (size_t)mm * a.N + n) = make_float4(o[0], o[1], o[2], o[3]);
                                if constexpr (PEER) {
                                    for (uint32_t g = 0; g < a.n_peers; ++g)
                                        if (a.peer_out[g] != a.out)
                                            *reinterpret_cast<float4*>(a.peer_out[g] + (size_t)mm * a.N + n) = make_float4(o[0], o[1], o[2], o[3]);
                                }
                            } else {
#pragma unroll
                                for (uint32_t k = 0; k < 4; ++k) a.out[tiled_out_offset(mm, n + k, a.layout)] = o[k];
                            }
                            if (a.acc_out) *reinterpret_cast<int4*>(a.acc_out + (size_t)mm * a.N + n) = val[c];
                        }
                    }
                }
                named_bar_sync(1, kEpiThreads);  // s_misc[2] is rewritten by the next item
                // the slice that finishes last re-arms the tile's counters for the next launch
                if (et == 0 && s_misc[2]) {
                    if (atomicAdd(ctr + 1, 1u) == p.split - 1) { ctr[0] = 0u; ctr[1] = 0u; }
                }
            }
        }
        tc_fence_before_sync();
        }
    }

    // ---------------- tear-down (also the way out after a wait that ran out)
    __syncthreads();
    if (*s_abort) {
        if (threadIdx.x == 0) {
            // Give B copies that may still be in flight time to land before the shared memory is
            // handed back: a TMA tile arrives within microseconds; wait a bounded ~100 us.
            const long long t0 = clock64();
            while (clock64() - t0 < 200000) {}
            atomicExch(p.dev_err, 2u);
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

size_t umma_smem_bytes(uint32_t n_tile, uint32_t a_slots, uint32_t b_slots, bool a_tmem) {
    return (size_t)(a_tmem ? 0 : a_slots) * kABytes + (size_t)b_slots * n_tile * kSlabK + kEpiWarps * kStageWarpBytes +
           kOneHotTabBytes + kNumBarriers * 8 + 16 + kEpiWarps * kBiasWarpBytes + 1024;
}
constexpr size_t kSmemLimit = 227 * 1024;
constexpr size_t kSmemOneCtaPerSm = 116 * 1024;  // of 228 KiB per SM

template <uint32_t N_TILE, bool A_TMEM, uint32_t SPS, bool PEER = false, bool EPI_TMA = false>
cudaError_t run(const CUtensorMap& map, const UmmaParams& p, uint32_t grid, size_t smem, cudaStream_t s, const CUtensorMap* out_map = nullptr) {
    auto k = lut_onehot_umma_kernel<N_TILE, A_TMEM, SPS, PEER, EPI_TMA>;
    // Never two of these CTAs on one SM: the second would sit in tcgen05.alloc until the first has
    // freed its tensor memory, and with split tiles the first may be waiting for the second's slice.
    // The grid is at most one CTA per SM, but while the preceding kernel still holds some SMs
    // (programmatic dependent launch) the block scheduler doubles CTAs up wherever two fit - which a
    // shallow ring with a single builder group does.  More than half an SM's shared memory rules it out.
    if (smem < kSmemOneCtaPerSm) smem = kSmemOneCtaPerSm;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((kFirstAgenWarp + 4 * p.groups + kEpiWarps) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k, map, p, out_map ? *out_map : map);  // (the third argument is read by EPI_TMA instances only)
}

// Ring depths.  One-hot slots: an even number (two warps issue alternate slabs); in tensor memory what the
// two accumulators leave of the 512 columns, 32 columns a slab; in shared memory as many as leave the
// LUT ring at least as deep.  LUT slots: whatever shared memory still holds.
void ring_depths(uint32_t n_tile, bool a_tmem, uint32_t want_b, uint32_t* a_slots, uint32_t* b_slots) {
    uint32_t sa = kMaxASlots;
    if (a_tmem) {
        const uint32_t room = (512u - 2 * n_tile) / 32u;
        if (sa > room) sa = room & ~1u;
    } else {
        while (sa > 2 && umma_smem_bytes(n_tile, sa, sa, false) > kSmemLimit) sa -= 2;
    }
    uint32_t sb = kMaxBSlots;
    while (sb > sa && umma_smem_bytes(n_tile, sa, sb, a_tmem) > kSmemLimit) --sb;
    if (want_b && want_b < sb) sb = want_b < 2 ? 2 : want_b;
    // Both rings hold an even number of slots: the two MMA-issuing warps take alternate slabs, so with an
    // even ring every slot is always consumed by the same warp, whose program order then guarantees that
    // a slot's previous use was waited for before the next one is asked about.  (An mbarrier parity wait
    // tells only two consecutive phases apart: asked about use q while use q-1 is still outstanding, it
    // answers for use q-2.)
    sb &= ~1u;
    if (sa > sb) sa = sb;
    *a_slots = sa;
    *b_slots = sb;
}
bool tile_ok(uint32_t n_tile, bool a_tmem) {
    if (a_tmem) return n_tile == 64 || n_tile == 128 || n_tile == 160 || n_tile == 192;
    return n_tile == 64 || n_tile == 128 || n_tile == 256;
}

}  // namespace

bool umma_supported(uint32_t CB, uint32_t CT, uint32_t N) {
    const bool ct_ok = CT == 8 || CT == 16 || CT == 32 || CT == 64 || CT == 128 || CT == 256;
    // CB % 16: a thread reads its row's indices with aligned vector loads; it also makes
    // CB*CT a multiple of 128, so there is no ragged slab
    return ct_ok && CB > 0 && CB % 16 == 0 && N > 0 && N % 16 == 0;
}

bool umma_tile_ok(uint32_t n_tile, bool a_tmem) { return tile_ok(n_tile, a_tmem); }

uint32_t umma_auto_split(uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, uint32_t n_tile, int sm_count) {
    const uint32_t slabs = (uint32_t)(((uint64_t)CB * CT + kSlabK - 1) / kSlabK);
    const uint32_t tiles = ((M + kMTile - 1) / kMTile) * ((N + n_tile - 1) / n_tile);
    uint32_t split = 1;
    if (tiles < (uint32_t)sm_count) {
        split = (uint32_t)sm_count / tiles;
        // keep at least 32 slabs per item: below that the fixed cost of an item and the summing of the
        // slices outweigh the shorter main loop (768 -> 768 at 1024 tokens: 48 slabs unsplit 22.3 us, three
        // slices of 16 slabs 23.8 us)
        const uint32_t max_split = slabs / 32 ? slabs / 32 : 1;
        if (split > max_split) split = max_split;
        if (split > 16) split = 16;
        if (split < 1) split = 1;
    }
    return split;
}

// Shape heuristics behind LUTAMM_VARIANT_AUTO (the tuner replaces them by measurement):
//  * plenty of tiles: A in tensor memory, 192-wide tiles (the widest that leaves tensor-memory columns
//    for the one-hot ring beside two accumulators; measured 7 % faster than A in shared memory with
//    256-wide tiles at 65536 x 4096 -> 16384, which stays available as a plan option);
//  * fewer tiles than SMs: 128-wide tiles and the codebook axis split across CTAs until the SMs are
//    covered.
// operand / n_tile / sps != 0 force that choice.
void umma_default_plan(uint32_t M, uint32_t CB, uint32_t CT, uint32_t N, int sm_count, uint32_t operand,
                       uint32_t n_tile, uint32_t sps, UmmaPlan* p) {
    const uint32_t tm = (M + kMTile - 1) / kMTile;
    auto tiles_for = [&](uint32_t nt) { return tm * ((N + nt - 1) / nt); };
    bool a_tmem;
    if (operand == 0 && n_tile == 0) {
        const uint32_t sms = (uint32_t)sm_count;
        a_tmem = true;
        if (N >= 192 && tiles_for(192) >= sms) n_tile = 192;
        // 128-wide tiles would need a second, mostly empty round while 192-wide ones fill most SMs once
        else if (N >= 192 && tiles_for(128) > sms && 4 * tiles_for(192) >= 3 * sms) n_tile = 192;
        else n_tile = N > 64 ? 128 : 64;
    } else if (operand == 0) {
        a_tmem = n_tile != 256;
    } else {
        a_tmem = operand == 2;
        if (n_tile == 0) n_tile = a_tmem ? (N >= 192 ? 192 : (N > 64 ? 128 : 64)) : (N >= 256 ? 256 : (N > 64 ? 128 : 64));
    }
    p->n_tile = n_tile;
    p->a_tmem = a_tmem ? 1u : 0u;
    p->split = umma_auto_split(M, CB, CT, N, n_tile, sm_count);
    p->stages = 0;
    p->groups = 0;
    p->sps = sps;  // 0: chosen at launch from the ring depth
    p->max_ctas = (uint32_t)sm_count;
    p->epilogue = 0;
}

cudaError_t umma_make_tmap(CUtensorMap* out, const int8_t* lut_t, uint32_t CB, uint32_t CT, uint32_t N,
                           uint32_t n_tile, const char** why) {
    *why = nullptr;
    if (!umma_supported(CB, CT, N)) { *why = "tcgen05 variant: needs num_centroid in {8,16,32,64,128,256}, num_codebook % 16 == 0, N % 16 == 0"; return cudaErrorInvalidValue; }
    if (n_tile != 64 && n_tile != 128 && n_tile != 160 && n_tile != 192 && n_tile != 256) { *why = "tcgen05 variant: N tile must be 64, 128, 160, 192 or 256"; return cudaErrorInvalidValue; }
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) { *why = "cuTensorMapEncodeTiled is not available from this driver"; return cudaErrorNotSupported; }
    const uint64_t Kg = (uint64_t)CB * CT;
    cuuint64_t dims[2] = {Kg, N};
    cuuint64_t strides[1] = {Kg};
    cuuint32_t box[2] = {kSlabK, n_tile};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(lut_t), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the transposed LUT map"; return cudaErrorInvalidValue; }
    return cudaSuccess;
}

// fp32 [M][N] row-major output as 32 x 32 blocks with the 128-byte swizzle the epilogue stages them in
static cudaError_t make_out_tmap(CUtensorMap* out, float* base, uint32_t M, uint32_t N, const char** why) {
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) { *why = "cuTensorMapEncodeTiled is not available from this driver"; return cudaErrorNotSupported; }
    cuuint64_t dims[2] = {N, M};
    cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *why = "cuTensorMapEncodeTiled failed for the output map"; return cudaErrorInvalidValue; }
    return cudaSuccess;
}

cudaError_t launch_umma(const LutArgs& a, const CUtensorMap& lut_t_map, const UmmaPlan& plan, int32_t* acc_scratch,
                        uint32_t* tile_counters, uint32_t* dev_err, cudaStream_t s, const char** why) {
    *why = nullptr;
    if (a.M == 0 || a.N == 0) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(a.idx) & 15u) { *why = "tcgen05 variant: the index buffer must be 16-byte aligned"; return cudaErrorInvalidValue; }
    const bool a_tmem = plan.a_tmem != 0;
    if (!tile_ok(plan.n_tile, a_tmem)) {
        *why = "tcgen05 variant: N tile must be 64, 128 or 256 (A in shared memory) or 64, 128 or 192 (A in tensor memory)";
        return cudaErrorInvalidValue;
    }
    UmmaParams p;
    p.a = a;
    p.slabs_total = (uint32_t)(((uint64_t)a.CB * a.CT + kSlabK - 1) / kSlabK);
    uint32_t split = plan.split ? plan.split : 1;
    if (split > p.slabs_total) split = p.slabs_total;
    p.slabs_per_item = (p.slabs_total + split - 1) / split;
    split = (p.slabs_total + p.slabs_per_item - 1) / p.slabs_per_item;  // no empty slices
    p.split = split;
    ring_depths(plan.n_tile, a_tmem, plan.stages, &p.a_slots, &p.b_slots);
    if (p.a_slots < 2 || p.b_slots < 2) { *why = "tcgen05 variant: this tile leaves room for fewer than two slabs in flight"; return cudaErrorInvalidValue; }
    p.a_slots_magic = (uint32_t)(((1ull << 32) + p.a_slots - 1) / p.a_slots);
    // slabs a builder group takes per turn
    uint32_t sps = plan.sps >= 2 ? 2u : 1u;  // one measured at least as fast as two on every benchmark shape
    if (sps > p.a_slots / 2 || plan.n_tile == 160) sps = 1;  // (160-wide tiles are built for one slab per turn)
    p.tiles_m = (a.M + kMTile - 1) / kMTile;
    p.tiles_n = (a.N + plan.n_tile - 1) / plan.n_tile;
    p.log2_ct = 0;
    while ((1u << p.log2_ct) < a.CT) ++p.log2_ct;
    p.acc_scratch = acc_scratch;
    p.tile_counters = tile_counters;
    p.dev_err = dev_err;
    // Every one-hot slot must always be filled by the same builder group, so that the group's program
    // order puts its wait for use q-1 of the slot before its wait for use q: an mbarrier parity wait tells
    // only two consecutive phases apart, and groups do not wait for one another - with the slots rotating
    // through the groups, one group two uses ahead of a stalled one would take the stalled group's
    // still-pending phase for its own and overwrite a slab that was never consumed.  Slab x goes to group
    // (x / sps) % groups and to slot x % slots, so the condition is slots % (groups * sps) == 0: take the
    // largest such group count not above the one asked for.
    p.groups = plan.groups ? (plan.groups > kMaxAgenGroups ? kMaxAgenGroups : plan.groups) : 4;
    // Two-slab turns are counted per item, slots over the CTA's whole slab sequence: after an item with
    // an odd number of slabs the pairs would straddle slots differently and the slots would change
    // hands, so a CTA that takes several items of which any is odd builds one slab per turn.
    const uint64_t items = (uint64_t)p.tiles_m * p.tiles_n * split;
    const uint32_t cap = plan.max_ctas ? plan.max_ctas : 148u;
    const uint32_t grid = (uint32_t)(items < cap ? items : cap);
    // With one tile per CTA every role reaches the end of its main loop at about the same time on every SM;
    // from there on only the epilogue runs, and the next kernel of the stream - the next operator's search, a
    // programmatic dependent - may as well be launched: its CTAs stage their centroids on whatever SMs are or
    // become free and then wait for this grid to complete (BERT-base step -2 % with a warm L2, -4 % with the
    // L2 evicted).  With several tiles per CTA the CTAs finish an item apart, the early CTAs of the next kernel
    // pile up on the SMs that are free first, and its load is skewed for good (BERT-large step +4 %): not there.
    p.early_trigger = (items <= cap) ? 1u : 0u;
    if (sps == 2 && items > grid && ((p.slabs_per_item & 1u) || (p.slabs_total & 1u))) sps = 1;
    while (p.groups > 1 && p.a_slots % (p.groups * sps) != 0) --p.groups;
    if (split > 1 && (!acc_scratch || !tile_counters)) { *why = "tcgen05 variant: split > 1 needs scratch"; return cudaErrorInvalidValue; }
    const size_t smem = umma_smem_bytes(plan.n_tile, p.a_slots, p.b_slots, a_tmem);
    if (a.n_peers) {
        // the exchange fused into the epilogue: built for the tiles the default plans use
        if (a.n_peers > kMaxPeers || a.layout.tiled) { *why = "tcgen05 variant: peer stores need row-major output and at most 8 GPUs"; return cudaErrorInvalidValue; }
        if (plan.n_tile == 192 && a_tmem && sps == 1) return run<192, true, 1, true>(lut_t_map, p, grid, smem, s);
        if (plan.n_tile == 128 && a_tmem && sps == 1) return run<128, true, 1, true>(lut_t_map, p, grid, smem, s);
        *why = "tcgen05 variant: peer stores are built for 128- and 192-wide tiles with the one-hot operand in tensor memory";
        return cudaErrorNotSupported;
    }
    {
        const bool eligible = !a.n_peers && split == 1 && !a.layout.tiled && !a.acc_out && a_tmem && sps == 1 &&
                              (plan.n_tile == 192 || plan.n_tile == 128) && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
        // A CTA with several tiles runs the epilogue beside the next tile's main loop, where every instruction it
        // issues lengthens the builders' latency chain: there the copy-engine form pays most (BERT-large step
        // -3 %); after a CTA's only tile it still shortens the tail a little (BERT-base step -1 %).
        if (eligible && plan.epilogue != 1) {
            CUtensorMap om;
            cudaError_t e = make_out_tmap(&om, a.out, a.M, a.N, why);
            if (e != cudaSuccess) return e;
            if (plan.n_tile == 192) return run<192, true, 1, false, true>(lut_t_map, p, grid, smem, s, &om);
            return run<128, true, 1, false, true>(lut_t_map, p, grid, smem, s, &om);
        }
    }
#define LUTAMM_UMMA_CASE(NT, TM, SP) \
    if (plan.n_tile == NT && a_tmem == TM && sps == SP) return run<NT, TM, SP>(lut_t_map, p, grid, smem, s);
    LUTAMM_UMMA_CASE(64, true, 1)
    LUTAMM_UMMA_CASE(64, true, 2)
    LUTAMM_UMMA_CASE(128, true, 1)
    LUTAMM_UMMA_CASE(128, true, 2)
    LUTAMM_UMMA_CASE(160, true, 1)
    LUTAMM_UMMA_CASE(192, true, 1)
    LUTAMM_UMMA_CASE(192, true, 2)
    LUTAMM_UMMA_CASE(64, false, 1)
    LUTAMM_UMMA_CASE(64, false, 2)
    LUTAMM_UMMA_CASE(128, false, 1)
    LUTAMM_UMMA_CASE(128, false, 2)
    LUTAMM_UMMA_CASE(256, false, 1)
    LUTAMM_UMMA_CASE(256, false, 2)
#undef LUTAMM_UMMA_CASE
    *why = "tcgen05 variant: this tile / operand / slabs-per-turn combination is not built";
    return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------- LUT [rows][cols] -> [cols][rows]
namespace {
__global__ void transpose_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, uint32_t rows,
                                    uint32_t cols) {
    __shared__ int8_t tile[64][65];
    const uint32_t r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (uint32_t i = threadIdx.y; i < 64; i += blockDim.y) {
        const uint32_t r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < rows && c < cols) ? in[(size_t)r * cols + c] : (int8_t)0;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.y; i < 64; i += blockDim.y) {
        const uint32_t c = c0 + i, r = r0 + threadIdx.x;
        if (c < cols && r < rows) out[(size_t)c * rows + r] = tile[threadIdx.x][i];
    }
}
}  // namespace

cudaError_t launch_transpose_lut(const int8_t* lut, int8_t* lut_t, uint32_t rows, uint32_t cols, cudaStream_t s) {
    dim3 block(64, 8), grid((cols + 63) / 64, (rows + 63) / 64);
    transpose_i8_kernel<<<grid, block, 0, s>>>(lut, lut_t, rows, cols);
    return cudaGetLastError();
}

}  // namespace lutamm
