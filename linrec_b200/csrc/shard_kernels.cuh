// Sequence sharding: one row is split over several GPUs ("shards", shard s owns the columns
// [s*L, (s+1)*L) of every row).  The reference is single-device, so nothing here has a counterpart
// there; the algebra is the pair operator of scan_core.cuh applied across shards.
//
// Pipeline on every rank:
//   1. local scan of the shard with a zero carry-in (the ordinary scan kernels with `open_start`),
//      which also leaves per row the pair (P, Y) of the whole shard in a carry record;
//   2. linrec_edges_kernel (backward only) adds the two elements the neighbours need:
//      c at the shard's scan-last element and y at its scan-first element;
//   3. the records of all shards are all-gathered (NCCL) into local memory;
//   4. a fix-up kernel folds the records of the shards that come earlier in scan order into the
//      carry v that enters this shard, and adds v * (running product of the coefficients) to the
//      shard's results.  The walk along a row stops as soon as the running value is exactly 0:
//      from there on every correction is exactly +0, so stopping changes no bit of the result.
//
// Carry records are fp32: forward 2 floats per row (P, Y); backward 4 floats (P, Y, c_edge, y_edge).
#pragma once
#include "scan_core.cuh"

namespace linrec {

struct FixupParams {
    void* out0;          // forward: y        backward: dx      (updated in place)
    void* out1;          // backward: dc      (updated in place)
    const void* c;
    const void* yin;     // backward: forward outputs
    const float* carries;   // [nshards][numseq][rec] gathered records
    long long numseq, seqlen, row_stride;
    int shard, nshards;
    int rec;             // floats per record: 2 forward, 4 backward
};

// Shards in scan order: ascending scans visit shard 0 first, descending scans the last shard first.
template <bool ASC>
__device__ __forceinline__ int shard_at(int n, int nshards) { return ASC ? n : nshards - 1 - n; }

// backward only: c at the shard's scan-last element, y at its scan-first element
template <typename ST, bool ASC>
__global__ void linrec_edges_kernel(const ST* c, const ST* y, float* records, long long numseq, long long seqlen,
                                    long long row_stride)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= numseq) return;
    const long long first = ASC ? 0 : seqlen - 1, last = ASC ? seqlen - 1 : 0;
    records[4 * r + 2] = Storage<ST>::to_float(c[r * row_stride + last]);
    records[4 * r + 3] = Storage<ST>::to_float(y[r * row_stride + first]);
}

// One CTA per row (grid-stride over rows).  Every thread handles V consecutive elements per step;
// a step covers NT*V elements in scan order.
template <typename ST, int NT, bool BWD, bool ASC>
__global__ void __launch_bounds__(NT) linrec_fixup_kernel(const FixupParams p)
{
    constexpr int V = 4, NW = NT / 32, STEP = NT * V;
    __shared__ float wprod[NW];
    __shared__ float v_in_s;
    const int tid = (int)threadIdx.x, lane = tid & 31, w = tid >> 5;
    // my position among the shards in scan order
    const int my_pos = ASC ? p.shard : p.nshards - 1 - p.shard;

    for (long long row = blockIdx.x; row < p.numseq; row += gridDim.x) {
        // ---- carry that enters this shard ---------------------------------------------------------
        if (tid == 0) {
            float v = 0.0f;
            int prev = -1;
            for (int n = 0; n < my_pos; ++n) {
                const int s = shard_at<ASC>(n, p.nshards);
                const float* rec = p.carries + ((long long)s * p.numseq + row) * p.rec;
                if (BWD && prev >= 0) v *= p.carries[((long long)prev * p.numseq + row) * p.rec + 2];
                v = fmaf(v, rec[0], rec[1]);
                prev = s;
            }
            if (BWD && prev >= 0) v *= p.carries[((long long)prev * p.numseq + row) * p.rec + 2];
            v_in_s = v;
        }
        __syncthreads();
        float v = v_in_s;
        const long long rb = row * p.row_stride;
        ST* o0 = reinterpret_cast<ST*>(p.out0) + rb;
        ST* o1 = BWD ? reinterpret_cast<ST*>(p.out1) + rb : nullptr;
        const ST* c = reinterpret_cast<const ST*>(p.c) + rb;
        const ST* y = BWD ? reinterpret_cast<const ST*>(p.yin) + rb : nullptr;
        const bool have_next = my_pos + 1 < p.nshards;

        // ---- walk the shard in scan order until the carried value is exactly zero ------------------
        for (long long base = 0; base < p.seqlen && v != 0.0f; base += STEP) {
            // scan position n (0-based within the shard) <-> memory index
            float cc[V], oo[V], ys[V];
            bool ok[V];
            long long idx[V];
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const long long n = base + (long long)tid * V + j;
                ok[j] = n < p.seqlen;
                idx[j] = ASC ? n : p.seqlen - 1 - n;
                float coef = 1.0f;
                if (ok[j]) {
                    if (!BWD) {
                        coef = Storage<ST>::to_float(c[idx[j]]);
                    } else if (n > 0) {
                        // coefficient of the scan predecessor; for n == 0 the neighbour shard's edge
                        // coefficient is already folded into v
                        coef = Storage<ST>::to_float(c[ASC ? idx[j] - 1 : idx[j] + 1]);
                    }
                    oo[j] = Storage<ST>::to_float(o0[idx[j]]);
                    if (BWD) ys[j] = (n + 1 < p.seqlen) ? Storage<ST>::to_float(y[ASC ? idx[j] + 1 : idx[j] - 1]) : 0.0f;
                } else {
                    oo[j] = 0.0f;
                    if (BWD) ys[j] = 0.0f;
                }
                cc[j] = coef;
            }
            // running products inside the thread, then across the block
            float pr[V];
            pr[0] = cc[0];
#pragma unroll
            for (int j = 1; j < V; ++j) pr[j] = pr[j - 1] * cc[j];
            float incl = pr[V - 1];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl *= t;
            }
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);
            if (lane == 0) excl = 1.0f;
            if (lane == 31) wprod[w] = incl;
            __syncthreads();
            float before = 1.0f, total = 1.0f;
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const float t = wprod[k];
                if (k < w) before *= t;
                total *= t;
            }
            const float zin = v * before * excl;   // value entering this thread's first element
#pragma unroll
            for (int j = 0; j < V; ++j) {
                if (ok[j]) {
                    const float z = zin * pr[j];
                    const float nv = oo[j] + z;
                    o0[idx[j]] = Storage<ST>::from_float(nv);
                    if (BWD) {
                        // dc = dx * y_successor; the scan-last element is finished after the walk
                        const float dcv = Storage<ST>::to_float(o1[idx[j]]);
                        o1[idx[j]] = Storage<ST>::from_float(fmaf(z, ys[j], dcv));
                    }
                }
            }
            v = v * total;
            __syncthreads();   // wprod is rewritten by the next step
        }
        if (BWD) {
            // the scan-last element multiplies with y of the NEXT shard's scan-first element, which
            // the local pass could not know
            __syncthreads();
            if (tid == 0 && have_next) {
                const int nxt = shard_at<ASC>(my_pos + 1, p.nshards);
                const float y_edge = p.carries[((long long)nxt * p.numseq + row) * p.rec + 3];
                const long long last = ASC ? p.seqlen - 1 : 0;
                o1[last] = Storage<ST>::from_float(Storage<ST>::to_float(o0[last]) * y_edge);
            }
        }
        __syncthreads();   // v_in_s is rewritten for the next row
    }
}

}  // namespace linrec
