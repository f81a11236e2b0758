// Sequence sharding: one row is split over several GPUs ("shards", shard s owns the columns
// [s*L, (s+1)*L) of every row).  The reference is single-device, so nothing here has a counterpart
// there; the algebra is the pair operator of scan_core.cuh applied across shards.
//
// Pipeline on every rank:
//   1. local scan of the shard with a zero carry-in (the ordinary scan kernels with `open_start`),
//      which also leaves per row the pair (P, Y) of the whole shard in a carry record;
//   2. backward only, by the same kernel: the record also takes the two elements the neighbours
//      need, c at the shard's scan-last element and y at its scan-first element;
//   3. the records of all shards are all-gathered (NCCL) into local memory;
//   4. a fix-up kernel folds the records of the shards that come earlier in scan order into the
//      carry v that enters this shard, and computes the head of the shard again from that carry.
//      The walk along a row stops as soon as v * (running product of the coefficients) is exactly
//      zero: from there on the local results are the true ones.
//
// Carry records are fp32: forward 2 floats per row (P, Y); backward 4 floats (P, Y, c_edge, y_edge).
#pragma once
#include "scan_core.cuh"

namespace linrec {

struct FixupParams {
    void* out0;          // forward: y        backward: dx      (the head of every row is written again)
    void* out1;          // backward: dc
    const void* in0;     // forward: x        backward: dy
    const void* c;
    const void* yin;     // backward: forward outputs
    const float* carries;   // [nshards][numseq][rec] gathered records
    long long numseq, seqlen, row_stride;
    int shard, nshards;
    int rec;             // floats per record: 2 forward, 4 backward
    const PeerTable* px; // with px_epoch != 0: the records are read from the other ranks' exchange buffers
    uint32_t px_epoch;   // (16-byte records; one flag per owner in this rank's buffer) instead of `carries`
    int super_chunks;    // > 1: the "shards" are consecutive rows of ONE tensor (a real row cut into this many
                         //      pieces, a power of two): row r is shard r % super_chunks of real row
                         //      r / super_chunks, and the records are indexed by row
    long long wait_budget;   // clock ticks a wait for a peer's record may last
    uint32_t* status;    // status word that receives kStatusPeerTimeout
};

// Where the record of (shard s, row) is in the gathered array.
__device__ __forceinline__ const float* fixup_record(const FixupParams& p, int s, long long row)
{
    if (p.super_chunks > 1) return p.carries + ((row & ~(long long)(p.super_chunks - 1)) + s) * p.rec;
    return p.carries + ((long long)s * p.numseq + row) * p.rec;
}

// Peer exchange: the record of (shard s, row), read from rank s's buffer once rank s has flagged its
// records of this epoch as complete (a wait that runs out of its budget sets the status bit and reads
// whatever is there).
__device__ __forceinline__ float4 fixup_record_from_peer(const FixupParams& p, int s, long long row)
{
    const PeerTable& t = *p.px;
    const int par = (int)(p.px_epoch & 1u);
    if (!wait_epoch_reached(px_flag(t, t.me, par, s), p.px_epoch, p.wait_budget)) atomicOr(p.status, kStatusPeerTimeout);
    return ld_relaxed_sys_f32x4(px_record(t, s, par, row));
}

// Writes the peer table into a (zeroed) exchange buffer.
struct PeerTableArg {
    PeerTable t;
};
__global__ void linrec_exchange_init_kernel(PeerTable* dst, const PeerTableArg a)
{
    if (threadIdx.x == 0) *dst = a.t;
}

// Shards in scan order: ascending scans visit shard 0 first, descending scans the last shard first.
template <bool ASC>
__device__ __forceinline__ int shard_at(int n, int nshards) { return ASC ? n : nshards - 1 - n; }

// The walk along a row goes on while the deviation d of the local results from the true ones (the
// entering carry times the product of the coefficients so far) still matters at a step boundary, where
// the true value is v and the local scan's value v - d:
//   * d exactly zero: every later correction is zero whatever the coefficients that follow are;
//   * |d| <= 2^-26 |v| (a quarter of an ulp of v, v finite): the local value IS the true one up to less
//     than the rounding error that any fp32 evaluation commits at that element (2^-24 |v|); whatever the
//     later coefficients do to it -- a stretch of |c| > 1 lets it grow back -- they do to that rounding
//     error as well.  For c ~ U(0.99, 1) this ends the walk after ~3.6 k elements instead of the ~20.6 k
//     that the product needs to underflow.
// A threshold on |d| alone (say, subnormal) would NOT do: it is safe only for |c| <= 1 from there on, and
// where the true values are themselves tiny (the decaying tail behind an impulse) d is all there is.
// NaN in d or v keeps walking.
__device__ __forceinline__ bool fixup_carry_alive(float d, float v)
{
    if (d == 0.0f) return false;
    return !(fabsf(v) <= 3.402823466e+38f && fabsf(d) <= 0x1p-26f * fabsf(v));
}

// Eight consecutive elements of a row as floats, memory order.  VEC: 16-byte loads (the caller has
// checked alignment), else element loads.  `m0` may address elements outside [0, seqlen) only when
// VEC is false, where every element is bounds-checked.
template <typename ST, bool VEC>
__device__ __forceinline__ void load8(const ST* row, long long m0, long long seqlen, float fill, float (&v)[8])
{
    if (VEC) {
        constexpr int PC = Storage<ST>::kPerChunk;
#pragma unroll
        for (int k = 0; k < 8 / PC; ++k) {
            const uint4 q = *reinterpret_cast<const uint4*>(row + m0 + k * PC);
            Storage<ST>::unpack(q, &v[k * PC]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long m = m0 + j;
            v[j] = (m >= 0 && m < seqlen) ? Storage<ST>::to_float(row[m]) : fill;
        }
    }
}

template <typename ST, bool VEC>
__device__ __forceinline__ void store8(ST* row, long long m0, long long seqlen, const float (&v)[8])
{
    if (VEC) {
        constexpr int PC = Storage<ST>::kPerChunk;
#pragma unroll
        for (int k = 0; k < 8 / PC; ++k) *reinterpret_cast<uint4*>(row + m0 + k * PC) = Storage<ST>::pack(&v[k * PC]);
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long m = m0 + j;
            if (m >= 0 && m < seqlen) row[m] = Storage<ST>::from_float(v[j]);
        }
    }
}

// What one thread needs for one step of the walk, in MEMORY order (8 consecutive elements).
template <bool BWD>
struct FixupStep {
    float a[8];              // additive term: x (forward) / dy (backward)
    float c[8];              // forward: c of the element; backward: c of the scan predecessor
    float ys[BWD ? 8 : 1];   // backward: y of the scan successor
    long long m0;            // memory index of element 0
};

// One CTA per row (grid-stride over rows).  The head of the row -- as far as the carry that enters it
// can still change a result -- is COMPUTED AGAIN from its operands with the true carry, not patched:
// every thread handles 8 consecutive elements per step, a step covers NT*8 elements in scan order and
// is a block scan of (Y, P) pairs like a tile of the scan kernels (thread aggregate, warp scan by
// shuffles, cross-warp fold through shared memory, rerun of the 8 elements from the true carry).  So
// each result is rounded to the storage type once, exactly as the unsharded scan rounds it; adding a
// correction to the stored local result would round 2-byte results twice, and where the correction
// cancels most of the local value that shows.  Same traffic as patching: forward reads x, c and writes
// y (patching read y, c), backward reads dy, c, y and writes dx, dc.  The operands of the next step are
// requested before the current step is worked on, so the walk runs at one DRAM round trip per step.
// (Two steps ahead, with three operand sets taking turns, was measured and lost: the registers cost
// more resident CTAs than the extra step in flight gives back; 128 threads per CTA beat 256.)
//
// The walk ends once the DIFFERENCE between the true and the local carry, d = v_in * (product of c so
// far), no longer matters (fixup_carry_alive): from there on the local results are the true ones.
template <typename ST, int NT, bool BWD, bool ASC, bool VEC>
__global__ void __launch_bounds__(NT) linrec_fixup_kernel(const FixupParams p)
{
    constexpr int V = 8, NW = NT / 32, STEP = NT * V;
    __shared__ Pair wagg[2][NW];
    __shared__ float v_in_s, y_edge_s;
    __shared__ float4 rec_s[kMaxPeers];
    const int tid = (int)threadIdx.x, lane = tid & 31, w = tid >> 5;
    const long long L = p.seqlen;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();   // the scan that left the local results and the records has completed

    for (long long row = blockIdx.x; row < p.numseq; row += gridDim.x) {
        const int shard = p.super_chunks > 1 ? (int)(row & (p.super_chunks - 1)) : p.shard;
        const int my_pos = ASC ? shard : p.nshards - 1 - shard;   // my rank among the shards in scan order
        // ---- carry that enters this shard ---------------------------------------------------------
        // v = sum over the earlier shards n of Y_n * (product of everything between shard n and this one),
        // gathered from the nearest shard backwards: the multiplier only shrinks for decaying
        // coefficients, and once it is exactly zero no earlier shard can contribute (with many shards
        // per row -- super-chunks -- the walk usually ends after one record).  Backward pass: between
        // two shards lies the coefficient at the earlier one's scan-last element (record word 2),
        // which the local scans treated as 1.
        // Peer exchange: lane n of the first warp fetches the record of the shard at scan position n
        // from its owner (all of a row's loads cross NVLink together), one more lane the record of
        // the next shard (its y at the scan-first element, needed by the backward pass below).
        if (p.px_epoch != 0u) {
            if (w == 0) {
                const bool earlier = lane < my_pos, next = BWD && lane == my_pos + 1 && lane < p.nshards;
                if (earlier || next) rec_s[lane] = fixup_record_from_peer(p, shard_at<ASC>(lane, p.nshards), row);
                __syncwarp();
                if (lane == 0) {
                    float v = 0.0f, m = 1.0f;
                    for (int n = my_pos - 1; n >= 0; --n) {
                        const float4 rec = rec_s[n];
                        if (BWD) m *= rec.z;
                        v = fmaf(rec.y, m, v);
                        m *= rec.x;
                        if (m == 0.0f) break;
                    }
                    v_in_s = v;
                    if (BWD && my_pos + 1 < p.nshards) y_edge_s = rec_s[my_pos + 1].w;
                }
            }
        } else if (tid == 0) {
            float v = 0.0f, m = 1.0f;
            for (int n = my_pos - 1; n >= 0; --n) {
                const volatile float* rec = fixup_record(p, shard_at<ASC>(n, p.nshards), row);
                if (BWD) m *= rec[2];
                v = fmaf(rec[1], m, v);
                m *= rec[0];
                if (m == 0.0f) break;
            }
            v_in_s = v;
            if (BWD && my_pos + 1 < p.nshards)
                y_edge_s = reinterpret_cast<const volatile float*>(fixup_record(p, shard_at<ASC>(my_pos + 1, p.nshards), row))[3];
        }
        __syncthreads();
        float v = v_in_s;    // true value that enters the next step
        float d = v;         // what the local scan (which started from zero) is off by at that point
        const long long rb = row * p.row_stride;
        ST* o0 = reinterpret_cast<ST*>(p.out0) + rb;
        ST* o1 = BWD ? reinterpret_cast<ST*>(p.out1) + rb : nullptr;
        const ST* in0 = reinterpret_cast<const ST*>(p.in0) + rb;
        const ST* c = reinterpret_cast<const ST*>(p.c) + rb;
        const ST* y = BWD ? reinterpret_cast<const ST*>(p.yin) + rb : nullptr;

        // operands of the step that starts at scan position `base`
        auto fetch = [&](long long base, FixupStep<BWD>& st) {
            const long long n0 = base + (long long)tid * V;          // first scan position of the thread
            st.m0 = ASC ? n0 : L - n0 - V;                            // lowest memory index of its 8 elements
            if (n0 >= L) return;                                      // nothing of this thread is in range
            load8<ST, VEC>(in0, st.m0, L, 0.0f, st.a);
            float cr[8];
            load8<ST, VEC>(c, st.m0, L, 1.0f, cr);
            if constexpr (!BWD) {
#pragma unroll
                for (int j = 0; j < 8; ++j) st.c[j] = cr[j];
            } else {
                float yr[8];
                load8<ST, VEC>(y, st.m0, L, 0.0f, yr);
                // neighbours just outside the 8 elements (0 / 1 beyond the shard: the edge factors are
                // folded into the carry and the scan-last dc is finished after the walk)
                const long long below = st.m0 - 1, above = st.m0 + V;
                const float c_below = below >= 0 ? Storage<ST>::to_float(c[below]) : 1.0f;
                const float c_above = above < L ? Storage<ST>::to_float(c[above]) : 1.0f;
                const float y_below = below >= 0 ? Storage<ST>::to_float(y[below]) : 0.0f;
                const float y_above = above < L ? Storage<ST>::to_float(y[above]) : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (ASC) {
                        st.c[j] = j == 0 ? c_below : cr[j - 1];
                        st.ys[j] = j == 7 ? y_above : yr[j + 1];
                    } else {
                        st.c[j] = j == 7 ? c_above : cr[j + 1];
                        st.ys[j] = j == 0 ? y_below : yr[j - 1];
                    }
                }
            }
        };

        FixupStep<BWD> cur, nxt;
        if (fixup_carry_alive(d, v)) fetch(0, cur);
        int par = 0;
        for (long long base = 0; base < L && fixup_carry_alive(d, v); base += STEP, par ^= 1) {
            if (base + STEP < L) fetch(base + STEP, nxt);
            const long long n0 = base + (long long)tid * V;
            // operands in scan order; identity elements outside the shard
            float cc[8], xx[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const int j = ASC ? jj : 7 - jj;
                const bool in = n0 + jj < L;
                cc[jj] = in ? cur.c[j] : 1.0f;
                xx[jj] = in ? cur.a[j] : 0.0f;
            }
            Pair inc = pair_identity();
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                inc.y = fmaf(inc.y, cc[jj], xx[jj]);
                inc.p *= cc[jj];
            }
#pragma unroll
            for (int dd = 1; dd < 32; dd <<= 1) {
                Pair far;
                far.y = __shfl_up_sync(0xffffffffu, inc.y, dd);
                far.p = __shfl_up_sync(0xffffffffu, inc.p, dd);
                if (lane >= dd) inc = combine(far, inc);
            }
            Pair ex;
            ex.y = __shfl_up_sync(0xffffffffu, inc.y, 1);
            ex.p = __shfl_up_sync(0xffffffffu, inc.p, 1);
            if (lane == 0) ex = pair_identity();
            if (lane == 31) wagg[par][w] = inc;
            __syncthreads();   // (the other half of wagg belongs to the previous step: no second barrier)
            Pair before = pair_identity(), total = pair_identity();
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const Pair t = wagg[par][k];
                if (k < w) before = combine(before, t);
                total = combine(total, t);
            }
            const Pair pre = combine(before, ex);        // what precedes this thread inside the step
            if (n0 < L) {
                float val = fmaf(v, pre.p, pre.y);       // true value that enters the thread's first element
                float r0[8], r1[BWD ? 8 : 1];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const int j = ASC ? jj : 7 - jj;
                    val = fmaf(val, cc[jj], xx[jj]);
                    r0[j] = val;
                    if constexpr (BWD) r1[j] = val * cur.ys[j];   // dc = dx * y at the scan successor
                }
                store8<ST, VEC>(o0, cur.m0, L, r0);
                if constexpr (BWD) store8<ST, VEC>(o1, cur.m0, L, r1);
            }
            v = fmaf(v, total.p, total.y);
            d *= total.p;
            cur = nxt;
        }
        if constexpr (BWD) {
            // the scan-last element multiplies with y of the NEXT shard's scan-first element, which
            // the local pass could not know
            __syncthreads();
            if (tid == 0 && my_pos + 1 < p.nshards) {
                const long long last = ASC ? L - 1 : 0;
                o1[last] = Storage<ST>::from_float(Storage<ST>::to_float(o0[last]) * y_edge_s);
            }
        }
        __syncthreads();   // v_in_s and wagg are rewritten for the next row
    }
    // Peer exchange: once every CTA of this rank is done reading, tell all ranks that the slots of
    // this epoch may be reused (they will be, two epochs from now).
    if (p.px_epoch != 0u && tid == 0) {
        const PeerTable& t = *p.px;
        __threadfence();
        uint32_t* done = reinterpret_cast<uint32_t*>(static_cast<char*>(t.base[t.me]) + px_done_offset(t.max_rows, t.nranks));
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0u;
            for (int i = 0; i < t.nranks; ++i) st_release_sys_u32(px_ack(t, i, t.me), p.px_epoch);
        }
    }
}

}  // namespace linrec
