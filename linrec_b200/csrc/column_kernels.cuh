// Scan along a non-last dimension without a transposed copy.
//
// The tensor is seen as (nb, seqlen, nchan), contiguous, and the recurrence runs along the MIDDLE
// axis: every (batch, channel) pair is its own sequence and neighbouring channels are neighbours in
// memory.  That is the `dim` argument of the reference's Python operator
// (linrec/impl/python/ops.py:8-14); the reference's CUDA operators only scan the last dimension
// (linrec/impl/cuda/linrec_pipe.cu:17-35) and its callers transpose.
//
// Layout of the work.  One thread owns one 4-byte channel word (one fp32 channel, or two adjacent
// 2-byte channels) and walks down the sequence with one fused multiply-add per element: no shuffles,
// no cross-thread scan.  A CTA of NT threads covers DC = NT * (4 / sizeof(ST)) channels; a "chunk" is
// LC consecutive sequence positions of those channels, brought in by ONE tiled bulk-tensor copy per
// operand (box = DC x LC x 1 of a rank-3 tensor map, no swizzle: consecutive threads read consecutive
// words of a row, which is free of bank conflicts) through a ring of S stages with mbarriers.  The
// result overwrites the input chunk in shared memory and leaves with a bulk-tensor store.
//
// The backward pass needs the coefficient of the scan predecessor and the output of the scan
// successor; along this axis those are simply the neighbouring ROWS, so the coefficient and output
// boxes are fetched one row up or down (the row coordinate of a bulk-tensor copy has no alignment
// rule) and rows outside the tensor arrive as zeros, which are exactly the boundary values.
//
// Parallelism along the sequence.  A "unit" is one (batch, channel group) column.  A column is cut
// into jobs of K chunks; job (g, u) has ticket g * units + u, tickets are handed out in increasing
// order, and a CTA works through the jobs it holds in order.  Inside a job the carry stays in a
// register.  Between jobs it travels through one 16-byte descriptor per channel:
//   K == chunks per column   one job per column, no descriptors at all (many columns);
//   K == 1                   decoupled look-back per THREAD (few columns): if the predecessor's
//                            inclusive value is not there yet, the thread publishes the aggregate of
//                            its chunk (which is still in shared memory), walks back over the
//                            predecessors, and re-runs the chunk from the true carry;
//   in between               a job waits (bounded) for its predecessor's inclusive value, which was
//                            handed out `units` tickets earlier.
#pragma once
#include "scan_core.cuh"

namespace linrec {

struct ColParams {
    long long nb, seqlen, nchan;
    int dtiles;            // channel groups per batch entry
    long long units;       // nb * dtiles
    int nq;                // chunks per column
    int k_chunks;          // chunks per job
    int gens;              // jobs per column
    long long njobs;       // units * gens
    uint32_t* header;      // workspace header (ticket, status, epoch, done)
    TileDesc* desc;        // [gens][units][DC] descriptors (unused when gens == 1)
    long long wait_budget;
    uint32_t first_ticket; // test hook: tickets start here
    int logc;              // 1: `c` holds logarithms (see ScanParams::logc)
    const void* c_raw;     // the coefficient tensor itself (logc backward: one word per thread and chunk)
};

template <typename ST, int NT, int LC, int S, bool BWD>
struct ColLayout {
    static constexpr int V = 4 / (int)sizeof(ST);        // channels per thread
    static constexpr int DC = NT * V;                    // channels per CTA
    static constexpr int NIN = BWD ? 3 : 2;
    static constexpr size_t kArrayBytes = (size_t)LC * NT * 4;
    static constexpr size_t kStageBytes = kArrayBytes * NIN;
    static constexpr size_t kDynSmem = kStageBytes * S + 1024;
    static_assert(kArrayBytes % 128 == 0, "stage arrays must keep 128-byte alignment");
};

// A 4-byte shared-memory word <-> the V channel values it holds.
template <typename ST>
struct ChanWord;
template <>
struct ChanWord<float> {
    __device__ static __forceinline__ void unpack(uint32_t w, float* v) { v[0] = __uint_as_float(w); }
    __device__ static __forceinline__ uint32_t pack(const float* v) { return __float_as_uint(v[0]); }
};
template <>
struct ChanWord<__nv_bfloat16> {
    __device__ static __forceinline__ void unpack(uint32_t w, float* v)
    {
        v[0] = __uint_as_float(w << 16);
        v[1] = __uint_as_float(w & 0xffff0000u);
    }
    __device__ static __forceinline__ uint32_t pack(const float* v)
    {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[0], v[1]);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <>
struct ChanWord<__half> {
    __device__ static __forceinline__ void unpack(uint32_t w, float* v)
    {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        v[0] = f.x;
        v[1] = f.y;
    }
    __device__ static __forceinline__ uint32_t pack(const float* v)
    {
        __half2 h = __floats2half2_rn(v[0], v[1]);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// Descriptor with the job generation in its fourth word.
__device__ __forceinline__ void col_publish(TileDesc* d, float y, float p, uint32_t state, uint32_t epoch, uint32_t gen)
{
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(d), "r"(__float_as_uint(y)),
                 "r"(__float_as_uint(p)), "r"((epoch << 2) | state), "r"(gen)
                 : "memory");
}

// Exclusive prefix of job `gen` of one channel: combination of the predecessors back to the nearest
// one that holds an inclusive value.  `d_prev` is the descriptor of generation gen-1, `stride` the
// distance between generations.  The descriptors are fetched a window of W at a time (independent
// loads, one round trip per window) and then combined nearest first.  Every poll is bounded; on
// expiry the status word is flagged and the walk ends with what it has.
__device__ __forceinline__ Pair col_lookback(const TileDesc* d_prev, long long stride, int gen, uint32_t epoch,
                                             long long budget, uint32_t* status)
{
    constexpr int W = 8;
    Pair acc = pair_identity();
    const TileDesc* d = d_prev;
    for (int k0 = gen - 1; k0 >= 0; k0 -= W, d -= (long long)W * stride) {
        uint4 w[W];
#pragma unroll
        for (int i = 0; i < W; ++i)
            w[i] = (k0 - i >= 0) ? desc_load(d - (long long)i * stride, epoch) : make_uint4(0u, 0u, 2u, 0u);
#pragma unroll
        for (int i = 0; i < W; ++i) {
            const int k = k0 - i;
            if (k < 0) return acc;
            if (w[i].z == 0u || w[i].w != (uint32_t)k) {
                const TileDesc* dk = d - (long long)i * stride;
                const long long t0 = clock64();
                unsigned ns = 32;
                while (true) {
                    w[i] = desc_load(dk, epoch);
                    if (w[i].z != 0u && w[i].w == (uint32_t)k) break;
                    if (clock64() - t0 > budget) {
                        w[i].z = 0u;
                        break;
                    }
                    __nanosleep(ns);
                    if (ns < 1024) ns <<= 1;
                }
            }
            if (w[i].z == 0u) {
                atomicOr(status, kStatusLookbackTimeout);
                return acc;
            }
            acc = combine(desc_pair(w[i]), acc);
            if (w[i].z == 2u) return acc;
        }
    }
    return acc;
}

struct ColItem {
    uint32_t ticket;   // 0xffffffff: no more work
    int q;             // chunk index inside the column, in scan order
    int g;             // job generation = ticket / units
    uint32_t u;        // column unit   = ticket % units
};

// Launched with NT + 32 threads: NT consumer threads (one channel word each) and one producer warp
// whose lane 0 issues every bulk copy.  The two sides meet only on mbarriers:
//   full[s]   the operands of the chunk in stage s have landed        (producer -> consumers)
//   done[s]   every consumer has written its results into stage s     (consumers -> producer)
// The producer then stores the stage, waits until the store has read it, and refills it, so that
// S-1 chunks are in flight while one is being scanned.  There is no block-wide barrier in the loop.
template <typename ST, int NT, int LC, int S, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT + 32) linrec_column_kernel(const __grid_constant__ CUtensorMap tm_in0,
                                                                const __grid_constant__ CUtensorMap tm_c,
                                                                const __grid_constant__ CUtensorMap tm_y,
                                                                const __grid_constant__ CUtensorMap tm_out0,
                                                                const __grid_constant__ CUtensorMap tm_out1,
                                                                const ColParams p)
{
    using L = ColLayout<ST, NT, LC, S, BWD>;
    constexpr int V = L::V, DC = L::DC;
    constexpr uint32_t kEnd = 0xffffffffu;
    static_assert(S >= 2, "the ring needs two stages");
    static_assert(DC <= 256, "a bulk-tensor box is at most 256 elements wide");

    extern __shared__ uint8_t dyn_smem[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~(uintptr_t)1023);
    auto buf = [&](int s, int a) { return reinterpret_cast<uint32_t*>(base + (size_t)s * L::kStageBytes + (size_t)a * L::kArrayBytes); };

    __shared__ __align__(8) uint64_t full[S];
    __shared__ __align__(8) uint64_t done[S];
    __shared__ ColItem items[S];
    __shared__ int abort_flag;

    const int tid = (int)threadIdx.x;
    const uint32_t epoch = read_epoch(p.header);
    const uint32_t njobs = (uint32_t)p.njobs;
    const uint32_t units = (uint32_t)p.units;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(&full[s], 1u);
            ptx::mbar_init(&done[s], (uint32_t)NT);
        }
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();

    auto coords = [&](const ColItem& it, int& x0, int& l0, int& b) {
        b = (int)(it.u / (uint32_t)p.dtiles);
        x0 = (int)(it.u % (uint32_t)p.dtiles) * DC;
        const int mq = ASC ? it.q : p.nq - 1 - it.q;   // chunk index in memory order
        l0 = mq * LC;
    };

    if (tid >= NT) {
        // ================================ producer warp =============================================
        if (tid != NT) return;
        ptx::prefetch_tensormap(&tm_in0);
        ptx::prefetch_tensormap(&tm_c);
        ptx::prefetch_tensormap(&tm_out0);
        if (BWD) {
            ptx::prefetch_tensormap(&tm_y);
            ptx::prefetch_tensormap(&tm_out1);
        }
        ColItem cur{kEnd, 0, 0, 0u};
        int qend = 0;
        bool first = true, drained = false;
        uint32_t end_at = kEnd;   // index of the first item that carries "no more work"
        for (uint32_t j = 0;; ++j) {
            const int s = (int)(j % S);
            if (j >= (uint32_t)S) {
                // item j-S lived in this stage: wait for its results, store them, wait for the store's reads
                if (end_at != kEnd && j - (uint32_t)S >= end_at) break;
                if (!ptx::mbar_wait_bounded(&done[s], ((j / S) - 1u) & 1u, p.wait_budget)) {
                    if (!abort_flag) atomicOr(p.header + 1, kStatusCopyTimeout);
                    abort_flag = 1;
                    break;
                }
                int x0, l0, b;
                coords(items[s], x0, l0, b);
                ptx::tma_store_3d(&tm_out0, buf(s, 0), x0, l0, b);
                if (BWD) ptx::tma_store_3d(&tm_out1, buf(s, 2), x0, l0, b);
                ptx::tma_commit_group();
                ptx::tma_wait_group_read<0>();
            }
            if (drained) continue;   // only stores are left
            if (cur.q >= qend) {
                // next job: with one job per column nobody waits for anybody and the first ticket of a
                // CTA is fixed; jobs that wait for their predecessor may only wait for a ticket that a
                // running CTA holds, so there every ticket comes from the counter
                const bool fixed = p.gens == 1;
                cur.ticket = (first && fixed) ? p.first_ticket + blockIdx.x
                                              : p.first_ticket + (fixed ? gridDim.x : 0u) + atomicAdd(p.header, 1u);
                first = false;
                if (cur.ticket >= njobs) {
                    drained = true;
                    end_at = j;
                    items[s].ticket = kEnd;
                    ptx::mbar_arrive(&full[s]);
                    continue;
                }
                cur.g = (int)(cur.ticket / units);
                cur.u = cur.ticket - (uint32_t)cur.g * units;
                cur.q = cur.g * p.k_chunks;
                qend = cur.q + p.k_chunks < p.nq ? cur.q + p.k_chunks : p.nq;
            }
            items[s] = cur;
            int x0, l0, b;
            coords(cur, x0, l0, b);
            ++cur.q;
            ptx::mbar_arrive_expect_tx(&full[s], (uint32_t)L::kStageBytes);
            ptx::tma_load_3d(buf(s, 0), &tm_in0, &full[s], x0, l0, b);
            // backward: coefficient of the scan predecessor, output of the scan successor = neighbouring rows
            ptx::tma_load_3d(buf(s, 1), &tm_c, &full[s], x0, BWD ? (ASC ? l0 - 1 : l0 + 1) : l0, b);
            if (BWD) ptx::tma_load_3d(buf(s, 2), &tm_y, &full[s], x0, ASC ? l0 + 1 : l0 - 1, b);
        }
        ptx::tma_wait_group<0>();
        finish_launch(p.header, epoch);
        return;
    }

    // ==================================== consumers ===================================================
    float carry[V];
#pragma unroll
    for (int v = 0; v < V; ++v) carry[v] = 0.0f;

    for (uint32_t it = 0;; ++it) {
        const int s = (int)(it % S);
        if (!ptx::mbar_wait_bounded(&full[s], (it / S) & 1u, p.wait_budget)) {
            atomicOr(p.header + 1, kStatusCopyTimeout);
            abort_flag = 1;
            break;
        }
        const ColItem item = items[s];
        if (item.ticket == kEnd) break;
        const int q = item.q, g = item.g;
        const bool job_first = q == g * p.k_chunks;
        const bool job_last = q == p.nq - 1 || q == (g + 1) * p.k_chunks - 1;
        uint32_t* bx = buf(s, 0);
        uint32_t* bc = buf(s, 1);
        uint32_t* by = buf(s, BWD ? 2 : 1);
        const long long gen_stride = (long long)units * DC;
        TileDesc* my_desc = p.desc + ((long long)g * units + item.u) * DC + tid * V;

        // forward: the coefficient of a sequence's first element is defined away
        // (linrec/impl/cuda/linrec_ref.cuh:63); backward it arrives as an out-of-range zero
        if (!BWD && q == 0) {
            // (every thread clears its own word of the row, so no synchronisation is needed)
            const int first_row = ASC ? 0 : (int)(p.seqlen - 1 - (long long)(p.nq - 1) * LC);
            bc[first_row * NT + tid] = p.logc ? Storage<ST>::kNegInfPair : 0u;
        }

        if (job_first) {
            bool have_carry = true;
#pragma unroll
            for (int v = 0; v < V; ++v) carry[v] = 0.0f;
            if (g > 0) {
                // the predecessor job of the same column was handed out `units` tickets earlier
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const uint4 w = desc_load(my_desc + v - gen_stride, epoch);
                    if (w.z == 2u && w.w == (uint32_t)(g - 1)) carry[v] = __uint_as_float(w.x);
                    else have_carry = false;
                }
            }
            if (!have_carry) {
                if (p.k_chunks == 1 && g < p.gens - 1) {
                    // decoupled: publish the aggregate of this chunk alone, then look back
                    Pair agg[V];
#pragma unroll
                    for (int v = 0; v < V; ++v) agg[v] = pair_identity();
#pragma unroll 8
                    for (int i = 0; i < LC; ++i) {
                        const int r = ASC ? i : LC - 1 - i;
                        float xv[V], cv[V];
                        ChanWord<ST>::unpack(bx[r * NT + tid], xv);
                        ChanWord<ST>::unpack(bc[r * NT + tid], cv);
                        if (p.logc) {
#pragma unroll
                            for (int v = 0; v < V; ++v) cv[v] = expf(cv[v]);
                        }
#pragma unroll
                        for (int v = 0; v < V; ++v) {
                            agg[v].y = fmaf(agg[v].y, cv[v], xv[v]);
                            agg[v].p *= cv[v];
                        }
                    }
#pragma unroll
                    for (int v = 0; v < V; ++v) col_publish(my_desc + v, agg[v].y, agg[v].p, 1u, epoch, (uint32_t)g);
                }
#pragma unroll
                for (int v = 0; v < V; ++v)
                    carry[v] = col_lookback(my_desc + v - gen_stride, gen_stride, g, epoch, p.wait_budget, p.header + 1).y;
            }
        }

        // logc backward: the shifted coefficient box lacks the OWN coefficient of the chunk's scan-last
        // row; every thread fetches its word of that row from global memory
        float own_edge[V];
#pragma unroll
        for (int v = 0; v < V; ++v) own_edge[v] = 0.0f;
        if (BWD && p.logc) {
            const int mq = ASC ? q : p.nq - 1 - q;
            const long long l_edge = (long long)mq * LC + (ASC ? LC - 1 : 0);
            const long long b = item.u / (uint32_t)p.dtiles;
            const long long ch = (long long)(item.u % (uint32_t)p.dtiles) * DC + (long long)tid * V;
            if (l_edge < p.seqlen && ch < p.nchan) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(
                    reinterpret_cast<const ST*>(p.c_raw) + (b * p.seqlen + l_edge) * p.nchan + ch);
                ChanWord<ST>::unpack(w, own_edge);
            }
        }

        // ---- the chunk itself: one fused multiply-add per element, results in place ----------------
        {
            float val[V];
#pragma unroll
            for (int v = 0; v < V; ++v) val[v] = carry[v];
#pragma unroll 8
            for (int i = 0; i < LC; ++i) {
                const int r = ASC ? i : LC - 1 - i;
                float xv[V], cv[V];
                ChanWord<ST>::unpack(bx[r * NT + tid], xv);
                ChanWord<ST>::unpack(bc[r * NT + tid], cv);
                if (p.logc) {
#pragma unroll
                    for (int v = 0; v < V; ++v) cv[v] = expf(cv[v]);
                }
#pragma unroll
                for (int v = 0; v < V; ++v) val[v] = fmaf(val[v], cv[v], xv[v]);
                bx[r * NT + tid] = ChanWord<ST>::pack(val);
                if (BWD) {
                    float yv[V], dc[V];
                    ChanWord<ST>::unpack(by[r * NT + tid], yv);
                    if (p.logc) {
                        // gradient with respect to the logarithm: times the element's OWN coefficient, which
                        // sits one row further along the scan in the shifted coefficient box
                        const int ro = ASC ? r + 1 : r - 1;
                        float co[V];
                        if (ro >= 0 && ro < LC) {
                            ChanWord<ST>::unpack(bc[ro * NT + tid], co);
                        } else {
#pragma unroll
                            for (int v = 0; v < V; ++v) co[v] = own_edge[v];
                        }
#pragma unroll
                        for (int v = 0; v < V; ++v) yv[v] *= expf(co[v]);
                    }
#pragma unroll
                    for (int v = 0; v < V; ++v) dc[v] = val[v] * yv[v];
                    by[r * NT + tid] = ChanWord<ST>::pack(dc);
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) carry[v] = val[v];
        }
        if (job_last && g < p.gens - 1) {
#pragma unroll
            for (int v = 0; v < V; ++v) col_publish(my_desc + v, carry[v], 0.0f, 2u, epoch, (uint32_t)g);
        }
        ptx::fence_proxy_async_smem();   // the results are read by the store engine
        ptx::mbar_arrive(&done[s]);
    }
}

}  // namespace linrec
