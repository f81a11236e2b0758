// The scan kernels.
//
//   linrec_tma_kernel      persistent CTAs, tiles handed out by an atomic ticket, operands brought
//                          in by tiled bulk-tensor copies (TMA, 128-byte swizzle) through an
//                          S-stage shared-memory ring with mbarriers, results staged in shared
//                          memory and written back with bulk-tensor stores.
//   linrec_async_kernel    same tile algebra for 16-byte aligned rows of whole 16-byte chunks that are
//                          not whole 128-byte lines: 16-byte cp.async into a ring of shared tiles.
//   linrec_generic_kernel  same tile algebra, but plain coalesced loads and stores with bounds
//                          checks: any length, any (element-aligned) pointer, any row stride.
//   linrec_seq_kernel      one thread walks one row (the slow, obviously-right operator that the
//                          reference exposes as linrec_ref: linrec/impl/cuda/linrec_ref.cuh:53-94).
//   linrec_row_f64_kernel  double precision: one CTA per row, the carry kept by the CTA.
//   linrec_row_kernel      rows of any alignment (odd lengths): one CTA per row, aligned 16-byte accesses.
//   linrec_fixup_kernel    sequence sharding: adds carry_in * running product of c to a shard.
//
// Replaces linrec/impl/cuda/linrec_pipe.cuh:8-143 and linrec/impl/cuda/linrec_tile.cuh:158-249.
#pragma once
#include <type_traits>

#include "scan_core.cuh"

namespace linrec {

// Ticket -> tile coordinates.
struct TileCoord {
    long long row;     // first row of the tile
    int q;             // chain: piece index in scan order
    int piece;         // chain: piece index in memory order
    int valid;         // slots of a row piece that lie inside the row (chain: of the tile; else the row length)
};

template <int T, bool ASC>
__device__ __forceinline__ TileCoord decode_ticket(const ScanParams& p, uint32_t tk)
{
    TileCoord tc;
    if (p.chain) {
        const uint32_t ns = (uint32_t)p.numseq;
        tc.q = (int)(tk / ns);
        tc.row = (long long)(tk - (uint32_t)tc.q * ns);
        tc.piece = ASC ? tc.q : p.chunks_per_row - 1 - tc.q;
        const long long left = p.seqlen - (long long)tc.piece * T;
        tc.valid = left < T ? (int)left : T;
    } else {
        tc.q = 0;
        tc.piece = 0;
        tc.row = (long long)tk * p.rows_per_tile;
        tc.valid = (int)p.seqlen;
    }
    return tc;
}

// Shared-memory words of the chain logic.
struct ChainShared {
    Pair tprefix;   // exclusive prefix of the current tile
    int early;      // 1: tprefix was known before the operands were even scanned
};

// Everything that happens between "operands are in registers" and "results are in registers",
// shared by both tile kernels.  `after_read` has to contain a block barrier after which the
// operand buffers and wagg may be reused; it is passed in because the pipelined kernel refills
// its ring at exactly that point.
//
// Chain mode.  The scan-last warp links the tile to its row.  Fast path: the predecessor's
// descriptor was fetched ahead of time (`probe`, loaded one iteration earlier while the previous
// tile was still being worked on) and already holds an inclusive value; then the exclusive prefix
// is in shared memory before the barrier and nobody waits for the look-back.  Slow path: publish
// the aggregate, walk back over the predecessors, one more barrier.  Either way the warp then
// fetches the descriptor that the NEXT tile (`next_tk`) will want.
template <typename ST, int E, int NT, bool BWD, bool ASC, typename AfterRead>
__device__ __forceinline__ void tile_scan(const ScanParams& p, const Geometry& g,
                                          const Operands<E, BWD>& op, const TileCoord& tc,
                                          uint32_t tk, uint32_t next_tk, uint32_t epoch, uint4& probe, Pair* wagg,
                                          ChainShared* cs, float (&o0)[E], float (&o1)[BWD ? E : 1],
                                          AfterRead&& after_read)
{
    constexpr int NW = NT / 32;
    const bool linker = p.chain && (g.ws == NW - 1);
    if (linker && g.lane == 0) {
        int early = 0;
        Pair tp = pair_identity();
        if (tc.q == 0) {
            early = 1;
        } else {
            if (probe.z != 2u) probe = desc_load(p.desc + ((long long)tk - p.numseq), epoch);
            if (probe.z == 2u) {
                tp = desc_pair(probe);
                early = 1;
            }
        }
        cs->tprefix = tp;
        cs->early = early;
    }
    const ThreadScan ts = scan_thread_and_warp<E, NT, BWD, ASC>(op, g, wagg);
    if (!after_read()) return;   // contains the block barrier; false = the CTA is bailing out
    const Pair wp = cross_warp_prefix<NW>(g, wagg);
    Pair pre = pair_identity();
    if (p.chain) {
        const bool early = cs->early != 0;
        if (linker) {
            const Pair bagg = combine(wp, wagg[NW - 1]);
            TileDesc* d = p.desc + tk;
            const bool last_piece = (tc.q == p.chunks_per_row - 1);
            Pair tp;
            if (early) {
                tp = cs->tprefix;
                if (g.lane == 0 && !last_piece) publish(d, combine(tp, bagg), 2u, epoch);
            } else {
                if (g.lane == 0 && !last_piece) publish(d, bagg, 1u, epoch);
                tp = lookback(p, epoch, (long long)tk, tc.q, g.lane);
                if (g.lane == 0) {
                    if (!last_piece) publish(d, combine(tp, bagg), 2u, epoch);
                    cs->tprefix = tp;
                }
            }
            if (g.lane == 0 && last_piece && (p.carry_out || p.px_epoch)) emit_record<ST, BWD, ASC>(p, tc.row, combine(tp, bagg));
            // fetch ahead what the next tile of this CTA will ask for
            probe = make_uint4(0u, 0u, 0u, 0u);
            if (next_tk < (uint32_t)p.ntiles && next_tk >= (uint32_t)p.numseq)
                probe = desc_load(p.desc + ((long long)next_tk - p.numseq), epoch);
        }
        if (!early) __syncthreads();
        pre = cs->tprefix;
    }
    if (g.need_wp) pre = combine(pre, wp);
    pre = combine(pre, ts.excl);
    if (!p.chain && (p.carry_out || p.px_epoch) && g.k == g.tpr - 1 && g.row_in_tile < p.rows_per_tile) {
        const long long row = tc.row + g.row_in_tile;
        if (row < p.numseq) emit_record<ST, BWD, ASC>(p, row, combine(pre, ts.agg));
    }
    apply_carry<E, BWD, ASC>(op, pre.y, o0, o1);
}

// =================================================================================================
//  Bulk-copy pipeline kernel
// =================================================================================================
template <typename ST, int E, int NT, int S, int OB, bool BWD>
struct TmaLayout {
    static constexpr int T = E * NT;
    static constexpr int NIN = BWD ? 3 : 2;
    static constexpr int NOUT = BWD ? 2 : 1;
    static constexpr size_t kTileBytes = (size_t)T * sizeof(ST);
    static constexpr size_t kDynSmem = kTileBytes * (S * NIN + OB * NOUT) + 1024;   // + alignment slack
    static_assert(kTileBytes % 1024 == 0, "tile buffers must keep 1024-byte alignment");
    // CTAs per SM the kernel is compiled for: what shared memory allows, up to a thread count that
    // leaves the register allocator what the pass needs (forward with 16 elements per thread: ~80
    // registers -> 768 threads; backward or 32 elements per thread: ~128 -> 512 threads)
    static constexpr int kFitSmem = (int)((size_t)232448 / (kDynSmem + 1024 + 512));
    static constexpr int kMaxThreads = (BWD || E >= 32) ? 512 : 768;
    static constexpr int kByThreads = kMaxThreads / NT < 1 ? 1 : kMaxThreads / NT;
    static constexpr int kMinBlocks = kFitSmem < 1 ? 1 : (kFitSmem < kByThreads ? kFitSmem : kByThreads);
};

template <typename ST, int E, int NT, int S, int OB, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT, (TmaLayout<ST, E, NT, S, OB, BWD>::kMinBlocks))
linrec_tma_kernel(const __grid_constant__ CUtensorMap tm_in0, const __grid_constant__ CUtensorMap tm_c,
                  const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_out0,
                  const __grid_constant__ CUtensorMap tm_out1, const ScanParams p)
{
    using L = TmaLayout<ST, E, NT, S, OB, BWD>;
    constexpr int T = L::T, NW = NT / 32, NIN = L::NIN, NOUT = L::NOUT;
    constexpr int EPL = 128 / (int)sizeof(ST);   // elements per 128-byte line
    constexpr int LINES = T / EPL;

    extern __shared__ uint8_t dyn_smem[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~(uintptr_t)1023);
    auto in_buf = [&](int s, int a) { return reinterpret_cast<ST*>(base + (size_t)(s * NIN + a) * L::kTileBytes); };
    auto out_buf = [&](int o, int a) {
        return reinterpret_cast<ST*>(base + (size_t)(S * NIN + o * NOUT + a) * L::kTileBytes);
    };

    __shared__ __align__(8) uint64_t full[S];
    __shared__ uint32_t tile_of_stage[S];
    __shared__ uint32_t halo[S][2];      // backward, chain mode: raw 4-byte words around the tile
    __shared__ Pair wagg[NW];
    __shared__ ChainShared chain_sh;
    __shared__ int abort_flag;

    const Geometry g = make_geometry<E, NT, ASC>(p);
    const int tid = g.t;
    // The thread that issues every bulk copy, draws the tickets and owns the bulk-store groups.  It
    // sits in the warp that comes FIRST in scan order, because the warp that comes last links the tile
    // to its row (publishes, looks back, fetches the next descriptor): one warp doing both would do
    // them one after the other.
    constexpr int boss = ASC ? 0 : NT - 32;
    const uint32_t ntiles = (uint32_t)p.ntiles;
    const bool with_halo = BWD && p.chain;
    const uint32_t stage_bytes =
        (uint32_t)NIN * (p.chain ? (uint32_t)L::kTileBytes
                                 : (uint32_t)(p.rows_per_tile * p.slots_per_row) * (uint32_t)sizeof(ST));

    ptx::grid_launch_dependents();
    if (tid == boss) {
#pragma unroll
        for (int s = 0; s < S; ++s) ptx::mbar_init(&full[s], with_halo ? 2u : 1u);
        abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tm_in0);
        ptx::prefetch_tensormap(&tm_c);
        ptx::prefetch_tensormap(&tm_out0);
        if (BWD) {
            ptx::prefetch_tensormap(&tm_y);
            ptx::prefetch_tensormap(&tm_out1);
        }
    }
    __syncthreads();
    // everything above is this CTA's own; from here on global memory is read and written
    ptx::grid_dependency_wait();
    const uint32_t epoch = read_epoch(p.header);
    if (p.px_epoch >= 3u && tid < 32) wait_for_slot_release(p.px, p.px_epoch, p.peer_wait_budget, p.header + 1, tid);

    // Issuing thread only: start the copies of ticket `tk` into ring slot `s`.
    auto issue = [&](int s, uint32_t tk) {
        const TileCoord tc = decode_ticket<T, ASC>(p, tk);
        const int c1 = tc.piece * LINES;
        const int c2 = (int)tc.row;
        if (with_halo) {
            // words just below and just above the piece; at a row end the edge value 0
            const ST* crow = reinterpret_cast<const ST*>(p.c) + tc.row * p.row_stride;
            const ST* yrow = reinterpret_cast<const ST*>(p.yin) + tc.row * p.row_stride;
            const long long lo = (long long)tc.piece * T - 1;
            const long long hi = (long long)tc.piece * T + T;
            const ST* csrc = ASC ? crow + lo : crow + hi;   // coefficient at the scan predecessor
            const ST* ysrc = ASC ? yrow + hi : yrow + lo;   // output at the scan successor
            const bool c_ok = ASC ? (lo >= 0) : (hi < p.seqlen);
            const bool y_ok = ASC ? (hi < p.seqlen) : (lo >= 0);
            // 4-byte copies from the 4-byte-aligned word that contains the element
            // (a coefficient that lies before an open shard start is 1; both halves for 2-byte storage)
            if (c_ok) ptx::cp_async_4(&halo[s][0], reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(csrc) & ~(uintptr_t)3));
            else halo[s][0] = !row_is_open<ASC>(p, tc.row) ? (p.logc ? Storage<ST>::kNegInfPair : 0u) : (p.logc ? 0u : Storage<ST>::kOnePair);
            if (y_ok) ptx::cp_async_4(&halo[s][1], reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(ysrc) & ~(uintptr_t)3));
            else halo[s][1] = 0u;
            ptx::cp_async_mbar_arrive_noinc(&full[s]);
        }
        ptx::mbar_arrive_expect_tx(&full[s], stage_bytes);
        ptx::tma_load_3d(in_buf(s, 0), &tm_in0, &full[s], 0, c1, c2);
        ptx::tma_load_3d(in_buf(s, 1), &tm_c, &full[s], 0, c1, c2);
        if (BWD) ptx::tma_load_3d(in_buf(s, 2), &tm_y, &full[s], 0, c1, c2);
    };

    // Tickets.  Rows that fit a tile never wait for another tile, so there the first S+1 tickets of a
    // CTA are fixed round-robin (ticket = round*grid + CTA): no trip to the counter before the first
    // copy starts.  Chained rows WAIT for their predecessors' descriptors, and a wait may only ever be
    // for a ticket that a running CTA holds: a fixed ticket can belong to a CTA that is not resident yet
    // (another kernel shares the GPU) and would then be waited for until the budget runs out.  So in
    // chain mode every ticket, the first ones included, comes from the counter: a ticket exists only
    // once a running CTA has drawn it, CTAs work through theirs in increasing order, and the oldest
    // unfinished ticket is therefore always being worked on.  (`fixed_first` restores the fixed start
    // for measurements.)  All later tickets come from the counter in both modes.
    //
    // "Lazy" mode (one ring slot; chosen when a handful of very long rows is all there is): a CTA holds
    // ONE ticket at a time and draws the next only when its tile is finished.  Holding tickets ahead is
    // what hides the load latency, but when consecutive tickets are consecutive pieces of the same row,
    // a ticket parked behind a tile that is itself waiting in its look-back stalls every CTA behind
    // it; with one ticket per CTA the oldest unfinished tiles are always the ones being worked on.
    const uint32_t grid = gridDim.x;
    const bool lazy = (S == 1) && p.lazy;
    const bool fixed = !p.chain || p.fixed_first;
    const uint32_t dyn_base = p.first_ticket + (fixed ? (lazy ? 1u : (uint32_t)(S + 1)) * grid : 0u);
    uint32_t next_ticket = 0;   // meaningful in the issuing thread only: ticket held one step ahead
    if (tid == boss) {
        for (int s = 0; s < S; ++s) {
            const uint32_t tk = fixed ? p.first_ticket + (uint32_t)s * grid + blockIdx.x : dyn_base + atomicAdd(p.header, 1u);
            tile_of_stage[s] = tk;
            if (tk < ntiles) issue(s, tk);
        }
        if (!lazy) next_ticket = fixed ? p.first_ticket + (uint32_t)S * grid + blockIdx.x : dyn_base + atomicAdd(p.header, 1u);
    }
    __syncthreads();

    uint4 probe = make_uint4(0u, 0u, 0u, 0u);   // look-ahead copy of the predecessor's descriptor
    uint32_t it = 0;
    for (;; ++it) {
        const int s = (int)(it % S);
        const uint32_t tk = tile_of_stage[s];
        if (tk >= ntiles) break;
        // with a ring of one slot the next ticket is not known yet at this point
        const uint32_t next_tk = S > 1 ? tile_of_stage[(it + 1) % S] : 0xffffffffu;
        const TileCoord tc = decode_ticket<T, ASC>(p, tk);

        if (!ptx::mbar_wait_bounded(&full[s], (it / S) & 1u, p.wait_budget)) {
            atomicOr(p.header + 1, kStatusCopyTimeout);
            abort_flag = 1;
        }

        const bool open = row_is_open<ASC>(p, tc.row);   // (super-chunks only exist in chain mode: one row per tile)
        float pred_c = open ? 1.0f : 0.0f, succ_y = 0.0f;
        if (with_halo) {
            // the halo word holds the element in its low or high half for 2-byte storage
            const uint32_t wc = halo[s][0], wy = halo[s][1];
            // 2-byte storage: the element below the piece has an odd index (upper half of its word),
            // the element above it an even one (lower half)
            pred_c = Storage<ST>::half_of_word(wc, ASC);
            if (p.logc) pred_c = expf(pred_c);   // boundary constants were stored as logarithms
            succ_y = Storage<ST>::half_of_word(wy, !ASC);
        }
        // The thread whose run holds the row's first element in scan order.  Scanning downwards, that
        // element is the last one INSIDE the row: in a ragged last piece it sits at slot valid-1, not at
        // the end of the tile (whole 128-byte lines make `valid` a multiple of E, so it is the last slot
        // of thread valid/E - 1).
        const bool zero_first =
            !open && (p.chain ? (tc.q == 0 && (ASC ? g.t == 0 : g.t == tc.valid / E - 1)) : (g.k == 0));

        bool alive = true;
        const int ob = (int)(it % OB);
        if constexpr (!BWD) {
            Operands<E, BWD> op;
            load_operands<ST, E, NT, BWD, ASC, true>(op, g, in_buf(s, 0), in_buf(s, 1), in_buf(s, 1), pred_c, succ_y,
                                                     tc.valid, zero_first, p.logc != 0);
            float o0[E], o1[1];
            tile_scan<ST, E, NT, BWD, ASC>(p, g, op, tc, tk, next_tk, epoch, probe, wagg, &chain_sh, o0, o1, [&]() -> bool {
                // the output buffer about to be reused must have been drained by its bulk store
                if (tid == boss) ptx::tma_wait_group_read<OB - 1>();
                __syncthreads();
                if (abort_flag) {
                    alive = false;
                    return false;
                }
                if (tid == boss && !lazy) {   // ring slot s is free again: refill it with the ticket drawn earlier
                    tile_of_stage[s] = next_ticket;
                    if (next_ticket < ntiles) issue(s, next_ticket);
                    next_ticket = dyn_base + atomicAdd(p.header, 1u);
                }
                return true;
            });
            if (!alive) break;
            store_run<ST, E>(out_buf(ob, 0), g.t, o0);
        } else {
            // Backward kernels only.  A whole warp in the fragment behind the last whole row of an
            // unchained tile (rows a little longer than half a tile: almost half the warps) holds no
            // element: it contributes the identity and keeps only its roles -- the barriers and, if it
            // has the issuing thread, the copies.  The slots it leaves unwritten lie outside the box of
            // the bulk store.  It is a path of its own (guarding the steps of the common path with a
            // flag instead cost chained scans a third of their speed), and the forward kernels keep
            // their one straight path: with this shape the compiler schedules the common path of the
            // backward kernels better (0-15 % over the length sweep, 2-byte storage most) and that of
            // the forward kernels worse (up to 10 %).
            auto after_read = [&]() -> bool {
                if (tid == boss) ptx::tma_wait_group_read<OB - 1>();   // as above
                __syncthreads();
                if (abort_flag) {
                    alive = false;
                    return false;
                }
                if (tid == boss && !lazy) {
                    tile_of_stage[s] = next_ticket;
                    if (next_ticket < ntiles) issue(s, next_ticket);
                    next_ticket = dyn_base + atomicAdd(p.header, 1u);
                }
                return true;
            };
            if (!p.chain && __all_sync(0xffffffffu, g.row_in_tile >= p.rows_per_tile)) {
                if (g.ls == 31) wagg[g.ws] = pair_identity();
                (void)after_read();
            } else {
                Operands<E, BWD> op;
                load_operands<ST, E, NT, BWD, ASC, true>(op, g, in_buf(s, 0), in_buf(s, 1), in_buf(s, 2), pred_c, succ_y,
                                                         tc.valid, zero_first, p.logc != 0);
                float o0[E], o1[E];
                tile_scan<ST, E, NT, BWD, ASC>(p, g, op, tc, tk, next_tk, epoch, probe, wagg, &chain_sh, o0, o1, after_read);
                if (alive) {
                    store_run<ST, E>(out_buf(ob, 0), g.t, o0);
                    store_run<ST, E>(out_buf(ob, 1), g.t, o1);
                }
            }
            if (!alive) break;
        }
        ptx::fence_proxy_async_smem();
        __syncthreads();
        if (tid == boss) {
            const int c1 = tc.piece * LINES;
            const int c2 = (int)tc.row;
            ptx::tma_store_3d(&tm_out0, out_buf(ob, 0), 0, c1, c2);
            if (BWD) ptx::tma_store_3d(&tm_out1, out_buf(ob, 1), 0, c1, c2);
            ptx::tma_commit_group();
            if (lazy) {   // the tile is done: only now take the next ticket and start its copies
                const uint32_t nt = dyn_base + atomicAdd(p.header, 1u);
                tile_of_stage[s] = nt;
                if (nt < ntiles) issue(s, nt);
            }
        }
        if (lazy) __syncthreads();   // the new ticket must be visible before the next round reads it
    }

    if (tid == boss) {
        if (abort_flag) {
            // best effort: let copies already in flight land before the CTA gives its memory back
            for (uint32_t j = 1; j < (uint32_t)S; ++j) {
                const uint32_t jt = it + j;
                if (tile_of_stage[jt % S] < ntiles)
                    (void)ptx::mbar_wait_bounded(&full[jt % S], (jt / S) & 1u, p.wait_budget);
            }
        }
        ptx::tma_wait_group<0>();
        finish_scan(p, epoch);
    }
}

// =================================================================================================
//  Any-alignment kernel
// =================================================================================================
template <typename ST, int E, int NT, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT) linrec_generic_kernel(const ScanParams p)
{
    constexpr int T = E * NT, NW = NT / 32;
    __shared__ __align__(1024) ST buf_in0[T];
    __shared__ __align__(1024) ST buf_c[T];
    __shared__ __align__(1024) ST buf_y[BWD ? T : 8];
    __shared__ float halo[2];
    __shared__ Pair wagg[NW];
    __shared__ ChainShared chain_sh;
    __shared__ uint32_t ticket_s;

    const Geometry g = make_geometry<E, NT, ASC>(p);
    const int tid = g.t;
    const uint32_t ntiles = (uint32_t)p.ntiles;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const uint32_t epoch = read_epoch(p.header);
    const ST* gin0 = reinterpret_cast<const ST*>(p.in0);
    const ST* gc = reinterpret_cast<const ST*>(p.c);
    const ST* gy = reinterpret_cast<const ST*>(p.yin);
    ST* gout0 = reinterpret_cast<ST*>(p.out0);
    ST* gout1 = reinterpret_cast<ST*>(p.out1);
    const int spr = p.chain ? T : p.slots_per_row;
    if (p.px_epoch >= 3u && tid < 32) wait_for_slot_release(p.px, p.px_epoch, p.peer_wait_budget, p.header + 1, tid);

    bool first_round = true;
    for (;;) {
        // rows that fit a tile: first ticket fixed (one per CTA), later ones from the counter; chained
        // rows wait for each other, so there every ticket is drawn (see linrec_tma_kernel)
        if (tid == 0) {
            const bool fixed = !p.chain || p.fixed_first;
            ticket_s = (first_round && fixed) ? p.first_ticket + blockIdx.x
                                              : p.first_ticket + (fixed ? gridDim.x : 0u) + atomicAdd(p.header, 1u);
        }
        first_round = false;
        __syncthreads();   // also: everybody has finished storing the previous tile
        const uint32_t tk = ticket_s;
        if (tk >= ntiles) break;
        const TileCoord tc = decode_ticket<T, ASC>(p, tk);
        const long long col0 = (long long)tc.piece * T;

        // ---- cooperative, coalesced load with identity fill ------------------------------------
        if (p.vec) {
            // 16-byte chunks: rows are 16-byte aligned and a whole number of chunks long, so a chunk
            // lies entirely inside or entirely outside its row
            constexpr int PC = Storage<ST>::kPerChunk;
            constexpr uint32_t kOne = Storage<ST>::kOnePair;
            const int cpr = spr / PC;
            const long long first_col = ASC ? 0 : p.seqlen - PC;   // chunk that holds the row's scan-first element
            for (int ci = tid; ci < T / PC; ci += NT) {
                const int j = p.chain ? 0 : ci / cpr;
                const long long col = p.chain ? col0 + (long long)ci * PC : (long long)(ci - j * cpr) * PC;
                const long long row = tc.row + j;
                const bool ok = (p.chain || j < p.rows_per_tile) && col < p.seqlen && row < p.numseq;
                const long long off = row * p.row_stride + col;
                const int phys = ci ^ ((ci >> 3) & 7);
                const uint32_t one = p.logc ? 0u : kOne;                          // identity coefficient
                const uint32_t zero = p.logc ? Storage<ST>::kNegInfPair : 0u;     // the coefficient 0
                uint4 q0 = make_uint4(0u, 0u, 0u, 0u), qc = make_uint4(one, one, one, one), qy = make_uint4(0u, 0u, 0u, 0u);
                if (ok) {
                    q0 = *reinterpret_cast<const uint4*>(gin0 + off);
                    qc = *reinterpret_cast<const uint4*>(gc + off);
                    if (BWD) qy = *reinterpret_cast<const uint4*>(gy + off);
                    if (!BWD && !p.open_start && col == first_col) {
                        if (ASC) qc.x = sizeof(ST) == 4 ? zero : ((qc.x & 0xffff0000u) | (zero & 0x0000ffffu));
                        else     qc.w = sizeof(ST) == 4 ? zero : ((qc.w & 0x0000ffffu) | (zero & 0xffff0000u));
                    }
                }
                reinterpret_cast<uint4*>(buf_in0)[phys] = q0;
                reinterpret_cast<uint4*>(buf_c)[phys] = qc;
                if (BWD) reinterpret_cast<uint4*>(buf_y)[phys] = qy;
            }
        } else {
            for (int i = tid; i < T; i += NT) {
                const int j = p.chain ? 0 : i / spr;
                const long long col = p.chain ? col0 + i : (long long)(i - j * spr);
                const long long row = tc.row + j;
                const bool ok = (p.chain || j < p.rows_per_tile) && col < p.seqlen && row < p.numseq;
                const long long off = row * p.row_stride + col;
                write_slot<ST>(buf_in0, i, ok ? Storage<ST>::to_float(gin0[off]) : 0.0f);
                float cv = ok ? Storage<ST>::to_float(gc[off]) : (p.logc ? 0.0f : 1.0f);
                // the coefficient of a row's very first element has no effect (closed rows only); with
                // padded rows that element need not be a thread's first slot, so it is cleared here
                if (!BWD && !p.open_start && col == (ASC ? 0 : p.seqlen - 1)) cv = p.logc ? -INFINITY : 0.0f;
                write_slot<ST>(buf_c, i, cv);
                if (BWD) write_slot<ST>(buf_y, i, ok ? Storage<ST>::to_float(gy[off]) : 0.0f);
            }
        }
        if (BWD && p.chain && tid < 2) {
            const long long lo = col0 - 1, hi = col0 + T;
            const long long rb = tc.row * p.row_stride;
            if (tid == 0) {   // coefficient at the scan predecessor of the piece
                const long long ci = ASC ? lo : hi;
                if (ci >= 0 && ci < p.seqlen) {
                    const float v = Storage<ST>::to_float(gc[rb + ci]);
                    halo[0] = p.logc ? expf(v) : v;
                } else {
                    halo[0] = p.open_start ? 1.0f : 0.0f;
                }
            } else {          // output at the scan successor of the piece
                const long long yi = ASC ? hi : lo;
                halo[1] = (yi >= 0 && yi < p.seqlen) ? Storage<ST>::to_float(gy[rb + yi]) : 0.0f;
            }
        }
        __syncthreads();

        const bool zero_first =
            !p.open_start && (p.chain ? (tc.q == 0 && g.s == 0) : (g.k == 0));
        Operands<E, BWD> op;
        load_operands<ST, E, NT, BWD, ASC, true>(op, g, buf_in0, buf_c, buf_y,
                                                  (BWD && p.chain) ? halo[0] : (p.open_start ? 1.0f : 0.0f),
                                                  (BWD && p.chain) ? halo[1] : 0.0f, tc.valid, zero_first, p.logc != 0);
        float o0[E], o1[BWD ? E : 1];
        uint4 probe = make_uint4(0u, 0u, 0u, 0u);   // no look-ahead here: the linking warp probes when it needs to
        tile_scan<ST, E, NT, BWD, ASC>(p, g, op, tc, tk, 0xffffffffu, epoch, probe, wagg, &chain_sh, o0, o1, [&]() -> bool {
            __syncthreads();
            return true;
        });
        // every thread holds its operands in registers, so the input buffers can take the results
        store_run<ST, E>(buf_in0, g.t, o0);
        if constexpr (BWD) store_run<ST, E>(buf_y, g.t, o1);
        __syncthreads();

        // ---- cooperative, coalesced store ------------------------------------------------------
        if (p.vec) {
            constexpr int PC = Storage<ST>::kPerChunk;
            const int cpr = spr / PC;
            for (int ci = tid; ci < T / PC; ci += NT) {
                const int j = p.chain ? 0 : ci / cpr;
                const long long col = p.chain ? col0 + (long long)ci * PC : (long long)(ci - j * cpr) * PC;
                const long long row = tc.row + j;
                const bool ok = (p.chain || j < p.rows_per_tile) && col < p.seqlen && row < p.numseq;
                if (ok) {
                    const long long off = row * p.row_stride + col;
                    const int phys = ci ^ ((ci >> 3) & 7);
                    *reinterpret_cast<uint4*>(gout0 + off) = reinterpret_cast<const uint4*>(buf_in0)[phys];
                    if (BWD) *reinterpret_cast<uint4*>(gout1 + off) = reinterpret_cast<const uint4*>(buf_y)[phys];
                }
            }
        } else {
            for (int i = tid; i < T; i += NT) {
                const int j = p.chain ? 0 : i / spr;
                const long long col = p.chain ? col0 + i : (long long)(i - j * spr);
                const long long row = tc.row + j;
                const bool ok = (p.chain || j < p.rows_per_tile) && col < p.seqlen && row < p.numseq;
                if (ok) {
                    const long long off = row * p.row_stride + col;
                    gout0[off] = Storage<ST>::from_float(read_slot<ST>(buf_in0, i));
                    if (BWD) gout1[off] = Storage<ST>::from_float(read_slot<ST>(buf_y, i));
                }
            }
        }
    }
    if (tid == 0) finish_scan(p, epoch);
}

// =================================================================================================
//  Asynchronous-copy kernel: rows that the bulk-copy kernel cannot take
// =================================================================================================
// Rows that are not whole 128-byte lines: every thread copies its share of a tile with cp.async
// straight into the swizzled layout through a ring of S tiles (the copies of the next S-1 tiles are
// in flight while tile i is scanned); padding chunks are written as identities.  Results go back
// through the same shared tile.  Same tile algebra and look-back as the other kernels.
//   CB = 16  rows 16-byte aligned and a whole number of 16-byte chunks long (L = 1000, 10000, ...);
//   CB = 4   rows 4-byte aligned and a whole number of 4-byte words long: every fp32 row whatever its
//            length or offset (L = 1001, views that start at an odd element), even-length rows of
//            2-byte elements.  One word per lane: a warp still moves whole 128-byte lines.
template <typename ST, int E, int NT, int S, bool BWD>
struct AsyncLayout {
    static constexpr int T = E * NT;
    static constexpr int NIN = BWD ? 3 : 2;
    static constexpr size_t kTileBytes = (size_t)T * sizeof(ST);
    static constexpr size_t kDynSmem = kTileBytes * S * NIN + 1024;
    // CTAs per SM the kernel is compiled for: what shared memory allows, up to a thread count that
    // leaves the register allocator what the pass needs
    static constexpr int kFitSmem = (int)((size_t)232448 / (kDynSmem + 1024 + 512));
    static constexpr int kMaxThreads = E >= 32 ? 384 : (BWD ? (sizeof(ST) == 2 ? 640 : 512) : 768);
    static constexpr int kByThreads = kMaxThreads / NT < 1 ? 1 : kMaxThreads / NT;
    static constexpr int kMinBlocks = kFitSmem < 1 ? 1 : (kFitSmem < kByThreads ? kFitSmem : kByThreads);
};

template <typename ST, int E, int NT, int S, int CB, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT, (AsyncLayout<ST, E, NT, S, BWD>::kMinBlocks)) linrec_async_kernel(const ScanParams p)
{
    using L = AsyncLayout<ST, E, NT, S, BWD>;
    static_assert(CB == 16 || CB == 4, "chunks are 16 or 4 bytes");
    constexpr int T = L::T, NW = NT / 32, NIN = L::NIN;
    constexpr int PC = CB / (int)sizeof(ST);          // elements per chunk
    constexpr uint32_t kOne = Storage<ST>::kOnePair;
    using Chunk = typename std::conditional<CB == 16, uint4, uint32_t>::type;
    extern __shared__ uint8_t dyn_smem[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~(uintptr_t)1023);
    auto buf = [&](int s, int a) { return reinterpret_cast<ST*>(base + (size_t)(s * NIN + a) * L::kTileBytes); };

    __shared__ uint32_t tile_of_stage[S];
    __shared__ uint32_t halo[S][2];
    __shared__ Pair wagg[NW];
    __shared__ ChainShared chain_sh;

    const Geometry g = make_geometry<E, NT, ASC>(p);
    const int tid = g.t;
    const uint32_t ntiles = (uint32_t)p.ntiles;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const uint32_t epoch = read_epoch(p.header);
    const ST* gin0 = reinterpret_cast<const ST*>(p.in0);
    const ST* gc = reinterpret_cast<const ST*>(p.c);
    const ST* gy = reinterpret_cast<const ST*>(p.yin);
    ST* gout0 = reinterpret_cast<ST*>(p.out0);
    ST* gout1 = reinterpret_cast<ST*>(p.out1);
    const int spr = p.chain ? T : p.slots_per_row;
    const int cpr = spr / PC;
    const bool with_halo = BWD && p.chain;
    if (p.px_epoch >= 3u && tid < 32) wait_for_slot_release(p.px, p.px_epoch, p.peer_wait_budget, p.header + 1, tid);

    // The chunks a thread copies are the same in every tile: chunk ci = tid + k*NT of the tile,
    // k = 0 .. CPT-1.  Where chunk ci lies -- its byte offset in the swizzled shared tile, its element
    // offset from the tile's first element, and the row of the tile it belongs to -- is found without
    // a division or a table: the thread keeps the place of its chunk 0 and steps from chunk to chunk.
    //   shared memory: the swizzle exchanges 16-byte chunks inside a 128-byte line by the line number
    //                  modulo 8; going from chunk ci to ci + NT moves a whole number of lines, and the
    //                  line number modulo 8 repeats with period one or two in k, so the offset of
    //                  chunk k is k*NT*CB plus one of two per-thread constants;
    //   global memory: chained rows: consecutive; rows that share a tile: (row, column) advance by
    //                  (NT / cpr, NT % cpr) chunks with at most one wrap into the next row.
    constexpr int CPT = T / PC / NT;   // chunks per thread and array
    auto chunk_offset = [](int ci) -> uint32_t {   // byte offset of chunk ci inside a swizzled tile buffer
        const uint32_t b = (uint32_t)ci * (uint32_t)CB;
        const uint32_t c16 = b >> 4;
        return ((c16 ^ ((c16 >> 3) & 7u)) << 4) | (b & 15u);
    };
    static_assert((NT * CB) % 1024 == 0 || (2 * NT * CB) % 1024 == 0, "the swizzle pattern must repeat within two steps");
    const uint32_t soff_even = chunk_offset(tid);
    const uint32_t soff_odd = chunk_offset(tid + NT) - (uint32_t)(NT * CB);
    int j0 = 0, col0 = tid, step_rows = 0, step_cols = 0;
    long long rel0 = (long long)tid * PC, step_rel = 0;
    if (!p.chain) {
        j0 = tid / cpr;
        col0 = tid - j0 * cpr;
        rel0 = (long long)j0 * p.row_stride + (long long)col0 * PC;
        step_rows = NT / cpr;
        step_cols = NT - step_rows * cpr;
        step_rel = (long long)step_rows * p.row_stride + (long long)step_cols * PC;
    }
    const long long wrap_rel = p.row_stride - (long long)cpr * PC;   // what a wrap into the next row adds
    // f(shared byte offset, element offset from the tile's first element, key); the chunk is inside the
    // tile's data iff key < lim (chain: key = column inside the tile; else key = row inside the tile)
    auto for_chunks = [&](auto&& f) {
        if (p.chain) {
#pragma unroll
            for (int k = 0; k < CPT; ++k)
                f((uint32_t)(k * NT * CB) + ((k & 1) ? soff_odd : soff_even), rel0 + (long long)k * NT * PC, (tid + k * NT) * PC);
        } else {
            int j = j0, col = col0;
            long long rel = rel0;
            // (the walk is the same for every tile; the empty volatile statement keeps the compiler from
            //  computing all CPT places once and holding them in registers across the tile loop, which
            //  measured slower even with four chunks per thread: the registers are worth more)
            asm volatile("" : "+r"(j), "+r"(col), "+l"(rel));
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                f((uint32_t)(k * NT * CB) + ((k & 1) ? soff_odd : soff_even), rel,
                  (j < p.rows_per_tile && col * PC < p.seqlen) ? j : 0x7fffffff);
                j += step_rows;
                col += step_cols;
                rel += step_rel;
                if (col >= cpr) {
                    col -= cpr;
                    ++j;
                    rel += wrap_rel;
                }
            }
        }
    };
    auto chunk_at = [&](int s_, int a, uint32_t soff) -> Chunk* {
        return reinterpret_cast<Chunk*>(reinterpret_cast<char*>(buf(s_, a)) + soff);
    };
    // tile -> (offset of its first element, bound that key[] has to stay under)
    auto tile_base = [&](const TileCoord& tc, int& lim) -> long long {
        const long long rows_left = p.numseq - tc.row;
        lim = p.chain ? tc.valid : (int)(rows_left < (long long)p.rows_per_tile ? rows_left : (long long)p.rows_per_tile);
        return tc.row * p.row_stride + (p.chain ? (long long)tc.piece * T : 0ll);
    };
    // every thread starts the copies of its chunks of ticket `tk` into ring slot `s`
    auto issue = [&](int s, uint32_t tk) {
        if (tk < ntiles) {
            const TileCoord tc = decode_ticket<T, ASC>(p, tk);
            int lim;
            const long long tb = tile_base(tc, lim);
            for_chunks([&](uint32_t soff, long long r, int ky) {
                const long long off = tb + r;
                Chunk* d0 = chunk_at(s, 0, soff);
                Chunk* d1 = chunk_at(s, 1, soff);
                if (ky < lim) {
                    if constexpr (CB == 16) {
                        ptx::cp_async_16(d0, gin0 + off);
                        ptx::cp_async_16(d1, gc + off);
                        if (BWD) ptx::cp_async_16(chunk_at(s, 2, soff), gy + off);
                    } else {
                        ptx::cp_async_4(d0, gin0 + off);
                        ptx::cp_async_4(d1, gc + off);
                        if (BWD) ptx::cp_async_4(chunk_at(s, 2, soff), gy + off);
                    }
                } else {
                    if constexpr (CB == 16) {
                        *d0 = make_uint4(0u, 0u, 0u, 0u);
                        *d1 = p.logc ? make_uint4(0u, 0u, 0u, 0u) : make_uint4(kOne, kOne, kOne, kOne);
                        if (BWD) *chunk_at(s, 2, soff) = make_uint4(0u, 0u, 0u, 0u);
                    } else {
                        *d0 = 0u;
                        *d1 = p.logc ? 0u : kOne;
                        if (BWD) *chunk_at(s, 2, soff) = 0u;
                    }
                }
            });
            if (with_halo && tid < 2) {
                const long long rb = tc.row * p.row_stride;
                const long long lo = (long long)tc.piece * T - 1, hi = (long long)tc.piece * T + T;
                // tid 0: coefficient at the scan predecessor of the piece; tid 1: output at its successor
                const long long idx = tid == 0 ? (ASC ? lo : hi) : (ASC ? hi : lo);
                const ST* src = (tid == 0 ? gc : gy) + rb + idx;
                if (idx >= 0 && idx < p.seqlen)
                    ptx::cp_async_4(&halo[s][tid], reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(src) & ~(uintptr_t)3));
                else
                    halo[s][tid] = tid == 1 ? 0u
                                   : p.open_start ? (p.logc ? 0u : kOne) : (p.logc ? Storage<ST>::kNegInfPair : 0u);
            }
        }
        ptx::cp_async_commit();   // one group per call, empty or not: the wait below counts groups
    };

    // Tickets as in the bulk-copy kernel: rows that fit a tile start from fixed round-robin tickets,
    // chained rows draw every ticket from the counter.  "Lazy" mode (a handful of very long rows): one
    // ticket at a time in ring slot 0, the next one drawn only when the tile has been scanned.
    const uint32_t grid = gridDim.x;
    const bool lazy = p.lazy != 0;
    const bool fixed = !p.chain || p.fixed_first;
    const uint32_t dyn_base = p.first_ticket + (fixed ? (lazy ? 1u : (uint32_t)(S + 1)) * grid : 0u);
    uint32_t next_ticket = 0;   // used by thread 0
    if (tid == 0) {
        for (int s = 0; s < S; ++s)
            tile_of_stage[s] = (lazy && s > 0) ? 0xffffffffu
                               : fixed ? p.first_ticket + (uint32_t)s * grid + blockIdx.x : dyn_base + atomicAdd(p.header, 1u);
        if (!lazy) next_ticket = fixed ? p.first_ticket + (uint32_t)S * grid + blockIdx.x : dyn_base + atomicAdd(p.header, 1u);
    }
    __syncthreads();
    for (int s = 0; s < S; ++s) issue(s, tile_of_stage[s]);

    uint4 probe = make_uint4(0u, 0u, 0u, 0u);   // look-ahead copy of the predecessor's descriptor
    for (uint32_t it = 0;; ++it) {
        const int s = lazy ? 0 : (int)(it % S);
        const uint32_t tk = tile_of_stage[s];
        if (tk >= ntiles) break;
        const uint32_t next_tk = lazy ? 0xffffffffu : tile_of_stage[(it + 1) % S];
        const TileCoord tc = decode_ticket<T, ASC>(p, tk);
        // this thread's copies of the tile have landed (the S-1 younger groups may still be in flight)
        if (lazy) ptx::cp_async_wait_group<0>();
        else ptx::cp_async_wait_group<S - 1>();
        __syncthreads();                     // ... and everybody else's

        float pred_c = p.open_start ? 1.0f : 0.0f, succ_y = 0.0f;
        if (with_halo) {
            pred_c = Storage<ST>::half_of_word(halo[s][0], ASC);
            if (p.logc) pred_c = expf(pred_c);   // boundary constants were stored as logarithms
            succ_y = Storage<ST>::half_of_word(halo[s][1], !ASC);
        }
        const bool zero_first = !p.open_start && (p.chain ? (tc.q == 0 && g.s == 0) : (g.k == 0));
        Operands<E, BWD> op;
        load_operands<ST, E, NT, BWD, ASC, true>(op, g, buf(s, 0), buf(s, 1), BWD ? buf(s, 2) : buf(s, 1), pred_c, succ_y,
                                                 tc.valid, zero_first, p.logc != 0);
        if (!BWD && !p.open_start && !ASC && !p.chain) {
            // padded rows scanned downwards: the row's first element in scan order is its last real
            // element, which need not be the last slot of a thread's run
            const int j = (int)p.seqlen - 1 - g.m * E;
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (e == j) op.c[e] = 0.0f;
        }
        if (!BWD && !p.open_start && !ASC && p.chain && tc.q == 0) {
            const int j = tc.valid - 1 - g.t * E;
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (e == j) op.c[e] = 0.0f;
        }
        float o0[E], o1[BWD ? E : 1];
        tile_scan<ST, E, NT, BWD, ASC>(p, g, op, tc, tk, next_tk, epoch, probe, wagg, &chain_sh, o0, o1, [&]() -> bool {
            __syncthreads();
            return true;
        });
        store_run<ST, E>(buf(s, 0), g.t, o0);
        if constexpr (BWD) store_run<ST, E>(buf(s, 2), g.t, o1);
        if (tid == 0) {
            if (lazy) {
                tile_of_stage[s] = dyn_base + atomicAdd(p.header, 1u);
            } else {   // the ticket drawn one tile ago; nobody waits for the counter's answer
                tile_of_stage[s] = next_ticket;
                next_ticket = dyn_base + atomicAdd(p.header, 1u);
            }
        }
        __syncthreads();
        {
            int lim;
            const long long tb = tile_base(tc, lim);
            for_chunks([&](uint32_t soff, long long r, int ky) {
                if (ky < lim) {
                    const long long off = tb + r;
                    *reinterpret_cast<Chunk*>(gout0 + off) = *chunk_at(s, 0, soff);
                    if (BWD) *reinterpret_cast<Chunk*>(gout1 + off) = *chunk_at(s, 2, soff);
                }
            });
        }
        __syncthreads();   // the slot has been read out: refill it
        issue(s, tile_of_stage[s]);
    }
    ptx::cp_async_wait_group<0>();
    if (tid == 0) finish_scan(p, epoch);
}

// =================================================================================================
//  Sequential operator: one thread per row
// =================================================================================================
template <typename ST, bool BWD>
__global__ void linrec_seq_kernel(const ScanParams p, int reverse)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= p.numseq) return;
    const long long L = p.seqlen;
    const long long rb = r * p.row_stride;
    const ST* in0 = reinterpret_cast<const ST*>(p.in0) + rb;
    const ST* c = reinterpret_cast<const ST*>(p.c) + rb;
    ST* out0 = reinterpret_cast<ST*>(p.out0) + rb;
    if (!BWD) {
        const bool asc = !reverse;
        float v = 0.0f;
        for (long long n = 0; n < L; ++n) {
            const long long i = asc ? n : L - 1 - n;
            const float x = Storage<ST>::to_float(in0[i]);
            float ci = Storage<ST>::to_float(c[i]);
            if (p.logc) ci = expf(ci);
            v = (n == 0) ? x : fmaf(v, ci, x);
            out0[i] = Storage<ST>::from_float(v);
        }
    } else {
        const ST* y = reinterpret_cast<const ST*>(p.yin) + rb;
        ST* out1 = reinterpret_cast<ST*>(p.out1) + rb;
        const bool asc = reverse != 0;   // the gradient scan runs against the forward direction
        float v = 0.0f;
        for (long long n = 0; n < L; ++n) {
            const long long i = asc ? n : L - 1 - n;
            const long long ip = asc ? i - 1 : i + 1;   // scan predecessor
            const long long is = asc ? i + 1 : i - 1;   // scan successor
            const float dy = Storage<ST>::to_float(in0[i]);
            float cp = (n == 0) ? 0.0f : Storage<ST>::to_float(c[ip]);
            if (p.logc && n > 0) cp = expf(cp);
            v = (n == 0) ? dy : fmaf(v, cp, dy);
            out0[i] = Storage<ST>::from_float(v);
            float ys = (n == L - 1) ? 0.0f : Storage<ST>::to_float(y[is]);
            if (p.logc) ys *= expf(Storage<ST>::to_float(c[i]));   // gradient with respect to the logarithm
            out1[i] = Storage<ST>::from_float(v * ys);
        }
    }
}


// The same walk in double precision: fp64 storage AND arithmetic (the type dispatch the reference
// leaves as a TODO, linrec/impl/cuda/linrec_pipe.cu:22).  Besides being an operator in its own right
// it is the GPU-side "exact" evaluation that fp32 results are judged against where two valid fp32
// evaluation orders already differ by more than the nominal tolerance.
template <bool BWD>
__global__ void linrec_seq_f64_kernel(const ScanParams p, int reverse)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= p.numseq) return;
    const long long L = p.seqlen;
    const long long rb = r * p.row_stride;
    const double* in0 = reinterpret_cast<const double*>(p.in0) + rb;
    const double* c = reinterpret_cast<const double*>(p.c) + rb;
    double* out0 = reinterpret_cast<double*>(p.out0) + rb;
    if (!BWD) {
        const bool asc = !reverse;
        double v = 0.0;
        for (long long n = 0; n < L; ++n) {
            const long long i = asc ? n : L - 1 - n;
            double ci = c[i];
            if (p.logc) ci = exp(ci);
            v = (n == 0) ? in0[i] : fma(v, ci, in0[i]);
            out0[i] = v;
        }
    } else {
        const double* y = reinterpret_cast<const double*>(p.yin) + rb;
        double* out1 = reinterpret_cast<double*>(p.out1) + rb;
        const bool asc = reverse != 0;   // the gradient scan runs against the forward direction
        double v = 0.0;
        for (long long n = 0; n < L; ++n) {
            const long long i = asc ? n : L - 1 - n;
            const long long ip = asc ? i - 1 : i + 1;   // scan predecessor
            const long long is = asc ? i + 1 : i - 1;   // scan successor
            double cp = (n == 0) ? 0.0 : c[ip];
            if (p.logc && n > 0) cp = exp(cp);
            v = (n == 0) ? in0[i] : fma(v, cp, in0[i]);
            out0[i] = v;
            double ys = (n == L - 1) ? 0.0 : y[is];
            if (p.logc) ys *= exp(c[i]);
            out1[i] = v * ys;
        }
    }
}

// =================================================================================================
//  Double precision: one CTA walks one row
// =================================================================================================
// fp64 storage and arithmetic for linrec_pipe / linrec_tile (the dtype dispatch that the reference leaves
// as a TODO, linrec/impl/cuda/linrec_pipe.cu:22) with the reference's own decomposition -- one CTA per
// row, the row taken tile by tile with the carry kept by the CTA (linrec/impl/cuda/linrec_pipe.cuh:8-70)
// -- so no look-back and no workspace: two doubles and a state would not fit the 16-byte descriptor word.
// A tile is 256 threads x 4 consecutive elements; per tile a thread folds its elements into a (Y, P)
// pair, the warp scans the pairs by shuffles, the warps' totals meet in shared memory (two sets taking
// turns: one barrier per tile), and every thread reruns its elements from the true value that enters
// them.  The next tile's operands are requested before the current tile is worked on.  Any row length,
// any 8-byte aligned pointer, any row stride (16-byte accesses where the layout allows them).  Rows are dealt to the CTAs round-robin: it needs a few
// hundred rows to fill the GPU, and the sequential operator remains the one for a handful of rows.
struct PairD {
    double y, p;
};
__device__ __forceinline__ PairD combine_d(PairD far, PairD near) { return PairD{fma(far.y, near.p, near.y), far.p * near.p}; }

template <bool BWD, bool ASC, bool VEC, bool LOGC>
__global__ void __launch_bounds__(256, BWD ? 2 : 4) linrec_row_f64_kernel(const ScanParams p)
{
    // VEC: every row starts on a 16-byte boundary and a thread's four elements do too (the host has
    // checked pointers, row stride and -- for descending scans -- an even row length): the unshifted
    // operands and the results go as 16-byte accesses.  LOGC: coefficients are given as logarithms.
    constexpr int NT = 256, E = 4, NW = NT / 32, T = NT * E;
    __shared__ PairD wagg[2][NW];
    const int tid = (int)threadIdx.x, lane = tid & 31, w = tid >> 5;
    const long long L = p.seqlen;
    int par = 0;   // runs on across rows, so that consecutive tiles never share a set of totals

    // What a thread requests for one tile: its own four elements of every operand as they lie in memory
    // (backward: plus the coefficient just before and the output just after its run in scan order, which
    // only a warp's edge lanes load themselves).  Nothing is computed from them until the tile is worked
    // on, so that the loads of the next tile stay in flight behind the arithmetic of the current one.
    struct Ops {
        double x[E], c[E], y[BWD ? E : 1], c_edge, y_edge;
    };
    for (long long row = blockIdx.x; row < p.numseq; row += gridDim.x) {
        const long long rb = row * p.row_stride;
        const double* in0 = reinterpret_cast<const double*>(p.in0) + rb;
        const double* c = reinterpret_cast<const double*>(p.c) + rb;
        const double* y = BWD ? reinterpret_cast<const double*>(p.yin) + rb : nullptr;
        double* out0 = reinterpret_cast<double*>(p.out0) + rb;
        double* out1 = BWD ? reinterpret_cast<double*>(p.out1) + rb : nullptr;

        // four consecutive elements of an array in SCAN order, starting at scan position n0
        auto load4 = [&](const double* a, long long n0, double (&v)[E], double fill) {
            if (VEC && n0 + E <= L) {
                const long long m0 = ASC ? n0 : L - n0 - E;
                const double2 lo = *reinterpret_cast<const double2*>(a + m0);
                const double2 hi = *reinterpret_cast<const double2*>(a + m0 + 2);
                v[ASC ? 0 : 3] = lo.x; v[ASC ? 1 : 2] = lo.y; v[ASC ? 2 : 1] = hi.x; v[ASC ? 3 : 0] = hi.y;
            } else {
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const long long n = n0 + j;
                    v[j] = n < L ? a[ASC ? n : L - 1 - n] : fill;
                }
            }
        };
        auto store4 = [&](double* a, long long n0, const double (&v)[E]) {
            if (VEC && n0 + E <= L) {
                const long long m0 = ASC ? n0 : L - n0 - E;
                *reinterpret_cast<double2*>(a + m0) = make_double2(v[ASC ? 0 : 3], v[ASC ? 1 : 2]);
                *reinterpret_cast<double2*>(a + m0 + 2) = make_double2(v[ASC ? 2 : 1], v[ASC ? 3 : 0]);
            } else {
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const long long n = n0 + j;
                    if (n < L) a[ASC ? n : L - 1 - n] = v[j];
                }
            }
        };

        auto fetch = [&](long long base, Ops& o) {
            const long long n0 = base + (long long)tid * E;
            load4(in0, n0, o.x, 0.0);
            load4(c, n0, o.c, LOGC ? 0.0 : 1.0);
            if constexpr (BWD) {
                load4(y, n0, o.y, 0.0);
                o.c_edge = 1.0;
                o.y_edge = 0.0;
                if (lane == 0 && n0 >= 1 && n0 - 1 < L) o.c_edge = c[ASC ? n0 - 1 : L - n0];
                if (lane == 31 && n0 + E < L) o.y_edge = y[ASC ? n0 + E : L - 1 - n0 - E];
            }
        };
        // The operands of the scan proper, in scan order.  Forward: the coefficient of an element is its
        // own (none for the row's first).  Backward: the coefficient at the scan PREDECESSOR's place and,
        // for d_coeffs, the output at the scan SUCCESSOR's place (linrec/impl/python/ops.py:32-40); the
        // neighbour just outside a thread's run comes from the adjacent lane by shuffle.  Beyond the
        // row: identity elements.
        auto prepare = [&](long long base, const Ops& o, double (&cc)[E], double (&ys)[BWD ? E : 1]) {
            const long long n0 = base + (long long)tid * E;
            if constexpr (!BWD) {
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    cc[j] = LOGC ? exp(o.c[j]) : o.c[j];
                    if (n0 + j == 0) cc[j] = 0.0;
                }
            } else {
                double c_pred = __shfl_up_sync(0xffffffffu, o.c[E - 1], 1);
                double y_succ = __shfl_down_sync(0xffffffffu, o.y[0], 1);
                if (lane == 0) c_pred = o.c_edge;
                if (lane == 31) y_succ = o.y_edge;
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const long long n = n0 + j;
                    double cp = j == 0 ? c_pred : o.c[j - 1];
                    if (LOGC) cp = exp(cp);
                    cc[j] = n == 0 ? 0.0 : (n < L ? cp : 1.0);
                    double yy = j == E - 1 ? y_succ : o.y[j + 1];
                    if (LOGC) yy *= exp(o.c[j]);   // gradient with respect to the logarithm
                    ys[j] = n < L - 1 ? yy : 0.0;
                }
            }
        };

        double carry = 0.0;   // the scan's value at the end of the previous tile
        Ops cur, nxt;
        fetch(0, cur);
        for (long long base = 0; base < L; base += T, par ^= 1) {
            if (base + T < L) fetch(base + T, nxt);
            double cc[E], ys[BWD ? E : 1];
            prepare(base, cur, cc, ys);
            PairD inc{0.0, 1.0};
#pragma unroll
            for (int j = 0; j < E; ++j) {
                inc.y = fma(inc.y, cc[j], cur.x[j]);
                inc.p *= cc[j];
            }
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                PairD far;
                far.y = __shfl_up_sync(0xffffffffu, inc.y, d);
                far.p = __shfl_up_sync(0xffffffffu, inc.p, d);
                if (lane >= d) inc = combine_d(far, inc);
            }
            PairD ex;
            ex.y = __shfl_up_sync(0xffffffffu, inc.y, 1);
            ex.p = __shfl_up_sync(0xffffffffu, inc.p, 1);
            if (lane == 0) ex = PairD{0.0, 1.0};
            if (lane == 31) wagg[par][w] = inc;
            __syncthreads();
            PairD pre{0.0, 1.0}, total{0.0, 1.0};
#pragma unroll
            for (int ww = 0; ww < NW; ++ww) {
                const PairD g = wagg[par][ww];
                if (ww < w) pre = combine_d(pre, g);
                total = combine_d(total, g);
            }
            pre = combine_d(pre, ex);
            double v = fma(carry, pre.p, pre.y);   // the true value that enters this thread's elements
            double r0[E], r1[BWD ? E : 1];
#pragma unroll
            for (int j = 0; j < E; ++j) {
                v = fma(v, cc[j], cur.x[j]);
                r0[j] = v;
                if constexpr (BWD) r1[j] = v * ys[j];
            }
            const long long n0 = base + (long long)tid * E;
            store4(out0, n0, r0);
            if constexpr (BWD) store4(out1, n0, r1);
            carry = fma(carry, total.p, total.y);
            cur = nxt;
        }
    }
}

// =================================================================================================
//  Rows of any alignment: one CTA walks one row with 16-byte accesses
// =================================================================================================
// Rows that start anywhere (odd lengths, sliced tensors) still lie in memory that can be read in
// aligned 16-byte chunks: a row is given to one CTA, which walks the aligned span around it -- `off`
// elements lie between the 16-byte boundary below the row start and the row start -- in tiles of
// NT threads x 8 elements with the carry kept by the CTA (the reference's decomposition,
// linrec/impl/cuda/linrec_pipe.cuh:8-70; no look-back, no workspace).  Elements of the span outside the
// row are identity elements and are never stored; a chunk none of whose elements belongs to the row is
// not read at all, and one that holds at least one element of the row lies in the same 16-byte word as
// that element, so no access leaves the memory of the tensor's own words.  All arrays of a call must
// share the row start's offset from a 16-byte boundary (the host checks it).  Otherwise the kernel is
// the double-precision one above with fp32 arithmetic: thread fold, warp scan by shuffles, totals
// through two sets of shared words (one barrier per tile), rerun from the true value; the next tile's
// chunks are requested before the current tile is worked on and nothing is computed from them until
// then.  It needs a few hundred rows to fill the GPU.
template <typename ST, int NT, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT) linrec_row_kernel(const ScanParams p)
{
    // a thread's run: 8 elements (two 16-byte chunks of fp32, one of 2-byte storage; 16 elements of 2-byte
    // storage per thread were measured and lost a quarter)
    constexpr int E = 8, PC = Storage<ST>::kPerChunk, NCH = E / PC, NW = NT / 32, T = NT * E;
    __shared__ Pair wagg[2][NW];
    const int tid = (int)threadIdx.x, lane = tid & 31, w = tid >> 5;
    const long long L = p.seqlen;
    const bool logc = p.logc != 0;
    int par = 0;   // runs on across rows, so that consecutive tiles never share a set of totals

    // What a thread requests for one tile, in MEMORY order: its E elements of every operand and
    // (backward, a warp's edge lanes only) the coefficient just before and the output just after its
    // run in scan order.
    struct Ops {
        float x[E], c[E], y[BWD ? E : 1], c_edge, y_edge;
    };
    for (long long row = blockIdx.x; row < p.numseq; row += gridDim.x) {
        const long long rb = row * p.row_stride;
        const ST* in0 = reinterpret_cast<const ST*>(p.in0) + rb;
        const ST* c = reinterpret_cast<const ST*>(p.c) + rb;
        const ST* y = BWD ? reinterpret_cast<const ST*>(p.yin) + rb : nullptr;
        ST* out0 = reinterpret_cast<ST*>(p.out0) + rb;
        ST* out1 = BWD ? reinterpret_cast<ST*>(p.out1) + rb : nullptr;
        // Positions v = 0, 1, ... count elements from the 16-byte boundary below the row start; element
        // e = v - off of the row lives at v.  The span is walked in whole runs of E positions.
        const int off = (int)((reinterpret_cast<uintptr_t>(in0) / sizeof(ST)) % PC);
        const long long Lv = (off + L + E - 1) / E * E;
        // lowest position of the run whose first element in scan order is scan position s0
        auto run_low = [&](long long s0) { return ASC ? s0 : Lv - s0 - E; };

        auto load_run = [&](const ST* a, long long v0, float fill, float (&o)[E]) {
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const long long vv = v0 + k * PC;
                if (vv + PC > off && vv < off + L) {
                    const uint4 q = *reinterpret_cast<const uint4*>(a + (vv - off));
                    Storage<ST>::unpack(q, &o[k * PC]);
                } else {
#pragma unroll
                    for (int i = 0; i < PC; ++i) o[k * PC + i] = fill;
                }
            }
        };
        auto store_run = [&](ST* a, long long v0, const float (&o)[E]) {
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const long long vv = v0 + k * PC;
                if (vv >= off && vv + PC <= off + L) {
                    *reinterpret_cast<uint4*>(a + (vv - off)) = Storage<ST>::pack(&o[k * PC]);
                } else {
#pragma unroll
                    for (int i = 0; i < PC; ++i) {
                        const long long e = vv + i - off;
                        if (e >= 0 && e < L) a[e] = Storage<ST>::from_float(o[k * PC + i]);
                    }
                }
            }
        };
        auto fetch = [&](long long base, Ops& o) {
            const long long v0 = run_low(base + (long long)tid * E);
            load_run(in0, v0, 0.0f, o.x);
            load_run(c, v0, 0.0f, o.c);
            if constexpr (BWD) {
                load_run(y, v0, 0.0f, o.y);
                o.c_edge = 1.0f;
                o.y_edge = 0.0f;
                // the neighbours just outside the run, at positions v0 - 1 and v0 + E
                const long long below = v0 - 1 - off, above = v0 + E - off;
                const long long ec = ASC ? below : above;      // scan predecessor of the run's first element
                const long long ey = ASC ? above : below;      // scan successor of its last element
                // (threads are in scan order either way: lane 0 has no predecessor lane, lane 31 no successor)
                if (lane == 0 && ec >= 0 && ec < L) o.c_edge = Storage<ST>::to_float(c[ec]);
                if (lane == 31 && ey >= 0 && ey < L) o.y_edge = Storage<ST>::to_float(y[ey]);
            }
        };

        float carry = 0.0f;   // the scan's value at the end of the previous tile
        Ops cur, nxt;
        fetch(0, cur);
        for (long long base = 0; base < Lv; base += T, par ^= 1) {
            if (base + T < Lv) fetch(base + T, nxt);
            const long long v0 = run_low(base + (long long)tid * E);
            // Operands of the scan proper, memory order: the coefficient applied to the carry that
            // enters a slot (forward: the element's own; backward: the one at its scan predecessor) and,
            // backward, the output at its scan successor (linrec/impl/python/ops.py:32-40).
            float cc[E], ys[BWD ? E : 1];
            if constexpr (!BWD) {
#pragma unroll
                for (int j = 0; j < E; ++j) cc[j] = logc ? expf(cur.c[j]) : cur.c[j];
            } else {
                // Threads are in scan order: lane - 1 holds the run that precedes in the scan (ascending:
                // the run below in memory, whose highest element is the neighbour; descending: the run
                // above, whose lowest element is), lane + 1 the run that follows.
                const float c_prev = __shfl_up_sync(0xffffffffu, cur.c[ASC ? E - 1 : 0], 1);
                const float y_next = __shfl_down_sync(0xffffffffu, cur.y[ASC ? 0 : E - 1], 1);
                const float c_pred_out = lane == 0 ? cur.c_edge : c_prev;
                const float y_succ_out = lane == 31 ? cur.y_edge : y_next;
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    float cp, yy;
                    if (ASC) {
                        cp = j == 0 ? c_pred_out : cur.c[j - 1];
                        yy = j == E - 1 ? y_succ_out : cur.y[j + 1];
                    } else {
                        cp = j == E - 1 ? c_pred_out : cur.c[j + 1];
                        yy = j == 0 ? y_succ_out : cur.y[j - 1];
                    }
                    if (logc) {
                        cp = expf(cp);
                        yy *= expf(cur.c[j]);   // gradient with respect to the logarithm
                    }
                    cc[j] = cp;
                    ys[j] = yy;
                }
            }
            // identity outside the row; nothing precedes the row's first element in scan order and
            // nothing follows its last
            float xx[E];
#pragma unroll
            for (int j = 0; j < E; ++j) xx[j] = cur.x[j];
            if (v0 - off <= 0 || v0 + E - off >= L) {   // only the runs at the ends of a row need any of this
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const long long e = v0 + j - off;
                    const bool inside = e >= 0 && e < L;
                    const bool first = ASC ? e == 0 : e == L - 1, last = ASC ? e == L - 1 : e == 0;
                    if (!inside) xx[j] = 0.0f;   // (a chunk that straddles the row's end holds a neighbour's elements)
                    if (!inside) cc[j] = 1.0f;
                    if (first) cc[j] = 0.0f;
                    if (BWD && (!inside || last)) ys[j] = 0.0f;
                }
            }
            Pair inc = pair_identity();
#pragma unroll
            for (int jj = 0; jj < E; ++jj) {
                const int j = ASC ? jj : E - 1 - jj;
                inc.y = fmaf(inc.y, cc[j], xx[j]);
                inc.p *= cc[j];
            }
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                Pair far;
                far.y = __shfl_up_sync(0xffffffffu, inc.y, d);
                far.p = __shfl_up_sync(0xffffffffu, inc.p, d);
                if (lane >= d) inc = combine(far, inc);
            }
            Pair ex;
            ex.y = __shfl_up_sync(0xffffffffu, inc.y, 1);
            ex.p = __shfl_up_sync(0xffffffffu, inc.p, 1);
            if (lane == 0) ex = pair_identity();
            if (lane == 31) wagg[par][w] = inc;
            __syncthreads();
            Pair pre = pair_identity(), total = pair_identity();
#pragma unroll
            for (int ww = 0; ww < NW; ++ww) {
                const Pair g = wagg[par][ww];
                if (ww < w) pre = combine(pre, g);
                total = combine(total, g);
            }
            pre = combine(pre, ex);
            float v = fmaf(carry, pre.p, pre.y);   // the true value that enters this thread's elements
            float r0[E], r1[BWD ? E : 1];
#pragma unroll
            for (int jj = 0; jj < E; ++jj) {
                const int j = ASC ? jj : E - 1 - jj;
                v = fmaf(v, cc[j], xx[j]);
                r0[j] = v;
                if constexpr (BWD) r1[j] = v * ys[j];
            }
            store_run(out0, v0, r0);
            if constexpr (BWD) store_run(out1, v0, r1);
            carry = fmaf(carry, total.p, total.y);
            cur = nxt;
        }
    }
}

}  // namespace linrec
