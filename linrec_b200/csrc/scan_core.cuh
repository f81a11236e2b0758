// Device-side building blocks of the linear-recurrence scan, shared by the bulk-copy (TMA)
// pipeline kernel and the any-alignment kernel.
//
// Replaces, from scratch, the reference's in-register block scan
// (linrec/impl/cuda/linrec_tile.cuh:33-114) and its tile loaders (linrec/impl/cuda/memio.cuh:12-198).
//
// Data model of one tile
// ----------------------
// A tile is T = E*NT "slots" held in shared memory, one array per operand.  Thread t owns the E
// consecutive slots [t*E, (t+1)*E).  Slots are stored in 16-byte chunks whose position inside
// each 128-byte line is XOR-ed with the line number modulo 8 -- exactly the layout the TMA unit
// produces with its 128-byte swizzle -- so that the per-thread 16-byte reads of a blocked
// arrangement are free of bank conflicts (8 consecutive threads hit 8 different chunk columns).
//
// A tile covers either a contiguous piece of ONE row ("chain" mode, rows longer than a tile, the
// pieces are linked by look-back carries) or several whole rows of `slots_per_row` slots each
// ("multi-row" mode).  In both modes a thread's slots never straddle two rows.
//
// Scan order.  ASC scans walk memory upwards, descending scans downwards; everything below is
// phrased in scan order (s = thread rank in scan order, k = number of threads of the same row
// that precede this thread inside the tile).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace linrec {

// ---- workspace layout ---------------------------------------------------------------------------
// Header words: [0] ticket counter, [1] status word (sticky until read), [2] epoch, [3] CTAs done.
// The workspace is zeroed ONCE by its owner; after that every launch cleans up after itself: the
// last CTA to finish resets the ticket and done counters and advances the epoch, and look-back
// descriptors carry the epoch they were written in, so stale ones read as "nothing yet".
constexpr int kHeaderBytes = 256;
constexpr uint32_t kStatusLookbackTimeout = 1u;
constexpr uint32_t kStatusCopyTimeout = 2u;
constexpr uint32_t kStatusPeerTimeout = 4u;

// One look-back descriptor per chained tile: 16 bytes that are always read and written with ONE
// 128-bit access, so that a reader sees the status together with the value it belongs to.
//   status = epoch * 4 + state;  a descriptor of another epoch counts as state 0
//   state 0  nothing yet
//   state 1  (y, p) is the aggregate of the tile alone
//   state 2  (y, p) is the inclusive value of the row up to and including the tile
struct __align__(16) TileDesc {
    float y, p;
    uint32_t status;
    uint32_t pad;
};

// ---- the associative operator -------------------------------------------------------------------
// A segment of the recurrence maps a carry-in v to  v*P + Y.  Composition "far then near":
//   (Y_f, P_f) o (Y_n, P_n) = (Y_f*P_n + Y_n, P_f*P_n);  identity (0, 1).
// (the reference's operator: linrec/impl/cuda/linrec_tile.cuh:53-54,74-75)
struct Pair {
    float y, p;
};
__device__ __forceinline__ Pair pair_identity() { return Pair{0.0f, 1.0f}; }
__device__ __forceinline__ Pair combine(Pair far, Pair near)
{
    return Pair{fmaf(far.y, near.p, near.y), far.p * near.p};
}

// ---- peer exchange (sequence sharding without a collective call) ------------------------------------
// Every rank owns one exchange buffer that all ranks of the node can address (peer-mapped memory).
// A rank's scan kernel leaves each row's record in its OWN buffer; the last of its CTAs to finish
// releases one flag in the buffer of EVERY rank ("my records of this epoch are complete").  The fix-up
// kernel of a rank waits on the flags in its own buffer and then READS the records it needs straight
// from the owners' buffers (one 16-byte load over NVLink per row and earlier shard, all of a row's
// loads in flight together, spread over all CTAs of the fix-up).  Pushing every record to every rank
// instead was measured: per row it costs the emitting CTA a system-scope fence, i.e. an NVLink round
// trip (8 % of the scan at 55 rows per CTA); in bulk from the last CTA it is a serial tail.
// Slots are double-buffered by the parity of the exchange epoch, and a rank acknowledges an epoch to
// all peers when its fix-up has finished, so that a slot is only overwritten (two epochs later)
// after every reader is done with it.
//   records [2][max_rows] x 16 B           (P, Y, c_edge, y_edge) of this rank's shard
//   flags   [2][nranks] x 4 B              epoch up to which rank i's records are complete
//   acks    [nranks] x 4 B                 last epoch rank i has finished reading
//   done    4 B                            fix-up CTAs finished (local bookkeeping)
// preceded by a 256-byte table of the peers' buffer addresses.
constexpr int kMaxPeers = 16;
constexpr size_t kPeerTableBytes = 256;
// Lives at the start of every exchange buffer (global memory, written once by the init call), so the
// kernels reach the peers through one pointer instead of carrying the table in their parameters.
struct PeerTable {
    void* base[kMaxPeers];   // base[i]: rank i's exchange buffer as mapped here (base[me] is this buffer)
    int nranks, me;
    long long max_rows;
};
static_assert(sizeof(PeerTable) <= kPeerTableBytes, "peer table must fit its slot");
__host__ __device__ inline size_t px_flags_offset(long long max_rows, int) { return kPeerTableBytes + (size_t)2 * max_rows * 16; }
__host__ __device__ inline size_t px_acks_offset(long long max_rows, int nranks)
{
    return (px_flags_offset(max_rows, nranks) + (size_t)2 * nranks * 4 + 255) / 256 * 256;
}
__host__ __device__ inline size_t px_done_offset(long long max_rows, int nranks) { return px_acks_offset(max_rows, nranks) + 256; }
__host__ __device__ inline size_t px_total_bytes(long long max_rows, int nranks) { return px_done_offset(max_rows, nranks) + 256; }
__device__ __forceinline__ float4* px_record(const PeerTable& t, int buf_of, int par, long long row)
{
    return reinterpret_cast<float4*>(static_cast<char*>(t.base[buf_of]) + kPeerTableBytes) + ((size_t)par * t.max_rows + row);
}
__device__ __forceinline__ uint32_t* px_flag(const PeerTable& t, int buf_of, int par, int from)
{
    return reinterpret_cast<uint32_t*>(static_cast<char*>(t.base[buf_of]) + px_flags_offset(t.max_rows, t.nranks)) +
           (par * t.nranks + from);
}
__device__ __forceinline__ uint32_t* px_ack(const PeerTable& t, int buf_of, int of_rank)
{
    return reinterpret_cast<uint32_t*>(static_cast<char*>(t.base[buf_of]) + px_acks_offset(t.max_rows, t.nranks)) + of_rank;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_relaxed_sys_f32x4(const float4* p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
// Bounded wait until *p has reached `target` (epochs only grow); false when the budget ran out.
__device__ __forceinline__ bool wait_epoch_reached(const uint32_t* p, uint32_t target, long long budget)
{
    if ((int32_t)(ld_acquire_sys_u32(p) - target) >= 0) return true;
    const long long t0 = clock64();
    unsigned ns = 64;
    while ((int32_t)(ld_acquire_sys_u32(p) - target) < 0) {
        if (clock64() - t0 > budget) return false;
        __nanosleep(ns);
        if (ns < 2048) ns <<= 1;
    }
    return true;
}

// ---- kernel parameters --------------------------------------------------------------------------
struct ScanParams {
    const void* in0;   // forward: x        backward: dy
    const void* c;     // coefficients
    const void* yin;   // backward only: outputs of the forward pass
    void* out0;        // forward: y        backward: dx
    void* out1;        // backward only: dc
    long long numseq, seqlen, row_stride;
    long long ntiles;
    int chain;           // 1: rows are longer than a tile and are chained
    int slots_per_row;   // multi-row mode: slots one row occupies (multiple of E)
    int rows_per_tile;   // multi-row mode
    int chunks_per_row;  // chain mode
    uint32_t* header;    // workspace header (ticket counter, status word)
    TileDesc* desc;      // chain mode: one descriptor per tile, zeroed before the launch
    long long wait_budget;  // clock ticks a wait inside this GPU may last (bulk copy, look-back)
    long long peer_wait_budget;   // clock ticks a wait for another rank may last (ranks start at different times)
    float* carry_out;    // optional: per row (P, Y) of the whole row, for sequence sharding
    int carry_stride;    // floats between the records of consecutive rows in carry_out
    int open_start;      // 1: the rows continue an earlier shard: the first coefficient counts, and a
                         //    coefficient that lies before the shard is taken as 1 (folded in later)
    int super_chunks;    // > 1 (a power of two; bulk-copy kernel, chained rows only): every real row was cut
                         //    into this many consecutive "rows" that are scanned independently; all but
                         //    the one that holds the real row's scan start are open (see open_start)
    uint32_t first_ticket;  // diagnostics: added to every ticket (0 in normal use)
    int vec;                // any-alignment kernel: rows allow 16-byte global accesses
    int lazy;               // bulk-copy kernel: draw the next ticket only when the current tile is finished
    int fixed_first;        // measurements only: chained rows also start from fixed round-robin tickets
    const PeerTable* px;    // sequence sharding: this rank's exchange buffer (its records are left there for all ranks)
    uint32_t px_epoch;      // epoch of this exchange; 0: no peer exchange in this launch (real epochs start at 1)
    int logc;               // 1: `c` holds logarithms; the loaders apply exp, the backward pass returns the
                            //    gradient with respect to the logarithm (d_c * c)
};

// Does `row` continue an earlier piece of its sequence (another GPU's shard, or the preceding
// super-chunk of the same real row)?
template <bool ASC>
__device__ __forceinline__ bool row_is_open(const ScanParams& p, long long row)
{
    if (p.super_chunks > 1) return ((int)row & (p.super_chunks - 1)) != (ASC ? 0 : p.super_chunks - 1);
    return p.open_start != 0;
}

// Storage helpers are declared further down; the record emitter needs them, so it follows them.

// ---- storage-type helpers -----------------------------------------------------------------------
template <typename ST>
struct Storage;

template <>
struct Storage<float> {
    static constexpr int kPerChunk = 4;
    __device__ static __forceinline__ void unpack(const uint4& q, float* v)
    {
        v[0] = __uint_as_float(q.x);
        v[1] = __uint_as_float(q.y);
        v[2] = __uint_as_float(q.z);
        v[3] = __uint_as_float(q.w);
    }
    __device__ static __forceinline__ uint4 pack(const float* v)
    {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                          __float_as_uint(v[3]));
    }
    __device__ static __forceinline__ float to_float(float v) { return v; }
    __device__ static __forceinline__ float from_float(float v) { return v; }
    static constexpr uint32_t kOnePair = 0x3f800000u;   // the value 1 as a 32-bit word
    static constexpr uint32_t kNegInfPair = 0xff800000u;   // -infinity (the logarithm of 0)
    __device__ static __forceinline__ float half_of_word(uint32_t w, bool) { return __uint_as_float(w); }
};

template <>
struct Storage<__nv_bfloat16> {
    static constexpr int kPerChunk = 8;
    __device__ static __forceinline__ void unpack(const uint4& q, float* v)
    {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ uint4 pack(const float* v)
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    static constexpr uint32_t kOnePair = 0x3f803f80u;   // the value 1 in both halves of a 32-bit word
    static constexpr uint32_t kNegInfPair = 0xff80ff80u;   // -infinity in both halves
    __device__ static __forceinline__ float half_of_word(uint32_t w, bool upper)
    {
        return __uint_as_float(upper ? (w & 0xffff0000u) : (w << 16));
    }
};

template <>
struct Storage<__half> {
    static constexpr int kPerChunk = 8;
    __device__ static __forceinline__ void unpack(const uint4& q, float* v)
    {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float* v)
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
    // the value 1 in both halves of a 32-bit word
    static constexpr uint32_t kOnePair = 0x3c003c00u;
    static constexpr uint32_t kNegInfPair = 0xfc00fc00u;   // -infinity in both halves
    // a 2-byte element held in the low / high half of a 32-bit word, as float
    __device__ static __forceinline__ float half_of_word(uint32_t w, bool upper)
    {
        const unsigned short bits = upper ? (unsigned short)(w >> 16) : (unsigned short)(w & 0xffffu);
        return __half2float(__ushort_as_half(bits));
    }
};

// Sequence sharding: the record of one row of this shard -- (P, Y) of the whole shard and, for the
// backward pass, c at the shard's scan-last element and y at its scan-first element (what the
// neighbouring shards need).  Written to the local record array and/or to this rank's exchange buffer,
// where the other ranks read it once publish_records() has told them that the launch is complete.
// (Deliberately NOT inlined and fed by value: it runs once per row; inlined into the tile loop its
// peer loop cost the backward kernel 37 registers and with them one resident CTA per SM.)
template <typename ST, bool BWD, bool ASC>
__device__ __noinline__ void emit_record(float* carry_out, int carry_stride, const PeerTable* px, uint32_t px_epoch,
                                         const ST* c, const ST* yin, long long seqlen, long long row_stride,
                                         long long row, float tot_p, float tot_y)
{
    float ce = 0.0f, ye = 0.0f;
    if (BWD) {
        const long long first = ASC ? 0 : seqlen - 1, last = ASC ? seqlen - 1 : 0;
        ce = Storage<ST>::to_float(c[row * row_stride + last]);
        ye = Storage<ST>::to_float(yin[row * row_stride + first]);
    }
    if (carry_out) {
        float* r = carry_out + carry_stride * row;
        r[0] = tot_p;
        r[1] = tot_y;
        if (BWD && carry_stride >= 4) {
            r[2] = ce;
            r[3] = ye;
        }
    }
    if (px_epoch != 0u) {
        const PeerTable& t = *px;
        const int par = (int)(px_epoch & 1u);
        *px_record(t, t.me, par, row) = make_float4(tot_p, tot_y, ce, ye);
    }
}

// Run by the thread that found its CTA to be the last of the launch: every record of this rank is then
// in its buffer (published by the writers' fences before they counted themselves done); one
// system-scope fence, then the flag in every rank's buffer.
static __device__ __noinline__ void publish_records(const PeerTable* px, uint32_t px_epoch)
{
    const PeerTable& t = *px;
    const int par = (int)(px_epoch & 1u);
    __threadfence_system();
    for (int r = 0; r < t.nranks; ++r) st_release_sys_u32(px_flag(t, r, par, t.me), px_epoch);
}

template <typename ST, bool BWD, bool ASC>
__device__ __forceinline__ void emit_record(const ScanParams& p, long long row, Pair tot)
{
    emit_record<ST, BWD, ASC>(p.carry_out, p.carry_stride, p.px, p.px_epoch, reinterpret_cast<const ST*>(p.c),
                              reinterpret_cast<const ST*>(p.yin), p.seqlen, p.row_stride, row, tot.p, tot.y);
}

// Before a launch writes records of epoch e it makes sure that every rank has acknowledged epoch
// e-2, whose slots it is about to overwrite (lanes 0..nranks-1 of the calling warp check one rank each).
static __device__ __noinline__ void wait_for_slot_release(const PeerTable* px, uint32_t px_epoch, long long budget,
                                                   uint32_t* status, int lane)
{
    if (lane < px->nranks) {
        if (!wait_epoch_reached(px_ack(*px, px->me, lane), px_epoch - 2u, budget)) atomicOr(status, kStatusPeerTimeout);
    }
}

// Byte offset of slot `i` inside a swizzled tile buffer (buffer base 1024-byte aligned).
template <typename ST>
__device__ __forceinline__ uint32_t slot_byte_offset(uint32_t i)
{
    const uint32_t b = i * (uint32_t)sizeof(ST);
    const uint32_t chunk = b >> 4;
    const uint32_t phys = chunk ^ ((chunk >> 3) & 7u);
    return (phys << 4) | (b & 15u);
}

template <typename ST>
__device__ __forceinline__ float read_slot(const ST* buf, int i)
{
    const char* p = reinterpret_cast<const char*>(buf) + slot_byte_offset<ST>((uint32_t)i);
    return Storage<ST>::to_float(*reinterpret_cast<const ST*>(p));
}

template <typename ST>
__device__ __forceinline__ void write_slot(ST* buf, int i, float v)
{
    char* p = reinterpret_cast<char*>(buf) + slot_byte_offset<ST>((uint32_t)i);
    *reinterpret_cast<ST*>(p) = Storage<ST>::from_float(v);
}

// Thread t's E slots, as E floats in memory order (16-byte shared loads, conflict free).
template <typename ST, int E>
__device__ __forceinline__ void load_run(const ST* buf, int t, float (&v)[E])
{
    constexpr int PC = Storage<ST>::kPerChunk;
    constexpr int CH = E / PC;
    static_assert(E % PC == 0, "a thread's run must be whole 16-byte chunks");
    const uint4* b4 = reinterpret_cast<const uint4*>(buf);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int cj = t * CH + j;
        const uint4 q = b4[cj ^ ((cj >> 3) & 7)];
        Storage<ST>::unpack(q, &v[j * PC]);
    }
}

template <typename ST, int E>
__device__ __forceinline__ void store_run(ST* buf, int t, const float (&v)[E])
{
    constexpr int PC = Storage<ST>::kPerChunk;
    constexpr int CH = E / PC;
    uint4* b4 = reinterpret_cast<uint4*>(buf);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int cj = t * CH + j;
        b4[cj ^ ((cj >> 3) & 7)] = Storage<ST>::pack(&v[j * PC]);
    }
}

// ---- per-thread geometry (does not change from tile to tile) ------------------------------------
struct Geometry {
    int t;            // thread index = memory rank of the thread's run inside the tile
    int s;            // thread rank in scan order
    int lane;         // hardware lane
    int ls;           // lane rank in scan order
    int ws;           // warp rank in scan order
    int m;            // memory rank of the run inside its row (multi-row) or tile (chain)
    int k;            // number of same-row threads that precede in scan order inside the tile
    int tpr;          // threads per row (multi-row) or NT (chain)
    int row_in_tile;  // multi-row: which row of the tile; chain: 0
    int start_warp;   // first warp (scan rank) that holds a piece of the row crossing into this warp
    bool need_wp;     // the thread's row began in an earlier warp
    bool has_excl;    // the scan-predecessor lane holds the same row
    bool lo_in_tile;  // slot just below the run belongs to the same row and tile
    bool hi_in_tile;  // slot just above the run belongs to the same row and tile
};

template <int E, int NT, bool ASC>
__device__ __forceinline__ Geometry make_geometry(const ScanParams& p)
{
    constexpr int NW = NT / 32;
    Geometry g;
    g.t = (int)threadIdx.x;
    g.lane = g.t & 31;
    const int w = g.t >> 5;
    g.ls = ASC ? g.lane : 31 - g.lane;
    g.ws = ASC ? w : NW - 1 - w;
    g.s = ASC ? g.t : NT - 1 - g.t;
    const int s = g.s;
    if (p.chain) {
        g.tpr = NT;
        g.m = g.t;
        g.k = s;
        g.row_in_tile = 0;
    } else {
        g.tpr = p.slots_per_row / E;
        g.row_in_tile = g.t / g.tpr;
        g.m = g.t - g.row_in_tile * g.tpr;
        g.k = ASC ? g.m : g.tpr - 1 - g.m;
    }
    g.lo_in_tile = g.m > 0;
    g.hi_in_tile = g.m < g.tpr - 1;
    g.has_excl = (g.ls >= 1) && (g.k >= 1);
    g.need_wp = g.k > g.ls;
    // k of the warp's scan-first lane tells where the row that crosses into this warp began
    const int k0 = __shfl_sync(0xffffffffu, g.k, ASC ? 0 : 31);
    // (threads past the last whole row of a multi-row tile form a fragment whose k may overshoot;
    //  their results are never stored, the clamp only keeps their reads inside the array)
    g.start_warp = max(0, (g.ws * 32 - k0) >> 5);
    return g;
}

// ---- operands of one thread ----------------------------------------------------------------------
template <int E, bool BWD>
struct Operands {
    float x[E];                 // additive term, memory order
    float c[E];                 // coefficient applied to the carry entering each slot
    float ysh[BWD ? E : 1];     // backward: forward output at the scan successor
};

// Reads the thread's operands from the tile buffers.
//   forward : x, c straight from the buffers.
//   backward: the coefficient of slot i is c at its scan PREDECESSOR and the multiplier for dc is
//             y at its scan SUCCESSOR (linrec/impl/python/ops.py:32-40).  For the slot at the end
//             of the thread's run the neighbour is the adjacent slot of the tile when that slot
//             belongs to the same row, otherwise the caller supplies it: `pred_c_outside` /
//             `succ_y_outside` are the halo words at a tile edge inside a row and the edge values
//             (0 unless the row continues on another shard) at a row end.
// `valid` is the number of slots of the thread's row piece that lie inside the row: the row length
// in multi-row mode (smaller than the slots a row occupies when rows are padded), and in chain mode
// the part of the tile before the row's end.  A neighbour slot at or beyond it is outside the row,
// so the caller's outside value is used for it as well.  With PATCH set, the coefficients of slots beyond it are
// forced to 1 AFTER the backward shift: padding must be an identity element (x = 0, c = 1) or the
// carry record of the row would pick up a stray factor (bulk copies fill with 0, and the shifted
// coefficient of the first padding slot is the row's last real coefficient).
// One coefficient read straight from the shared tile (the neighbour across a warp edge).
template <typename ST>
__device__ __forceinline__ float edge_coeff(const ST* b_c, int slot, bool logc)
{
    const float v = read_slot<ST>(b_c, slot);
    return logc ? expf(v) : v;
}

template <typename ST, int E, int NT, bool BWD, bool ASC, bool PATCH>
__device__ __forceinline__ void load_operands(Operands<E, BWD>& op, const Geometry& g,
                                              const ST* b_in0, const ST* b_c, const ST* b_y,
                                              float pred_c_outside, float succ_y_outside, int valid,
                                              bool zero_first, bool logc = false)
{
    load_run<ST, E>(b_in0, g.t, op.x);
    float craw[E];
    load_run<ST, E>(b_c, g.t, craw);
    // Coefficients given as logarithms: everything read from the coefficient tile goes through exp
    // (pred_c_outside is a coefficient already).
    if (logc) {
#pragma unroll
        for (int j = 0; j < E; ++j) craw[j] = expf(craw[j]);
    }
    const int a = g.t * E;          // first slot of the run inside the tile
    const int ra = g.m * E;         // ... and inside its row piece
    if (!BWD) {
#pragma unroll
        for (int j = 0; j < E; ++j) op.c[j] = craw[j];
    } else {
        float yraw[E];
        load_run<ST, E>(b_y, g.t, yraw);
        const int lo = a - 1, hi = a + E;
        // The neighbour just outside the run is the adjacent thread's edge element: it comes over a
        // warp shuffle (lane stride of a blocked run would make a direct shared read a 4-way bank
        // conflict); only the lane at the warp's edge reads shared memory.
        const bool lo_ok = g.lo_in_tile;
        const bool hi_ok = g.hi_in_tile && ra + E < valid;
        if (ASC) {   // predecessor = slot below, successor = slot above
            const float c_from_below = __shfl_up_sync(0xffffffffu, craw[E - 1], 1);
            const float y_from_above = __shfl_down_sync(0xffffffffu, yraw[0], 1);
            const float c_pred = !lo_ok ? pred_c_outside : (g.lane > 0 ? c_from_below : edge_coeff<ST>(b_c, lo, logc));
            const float y_succ = !hi_ok ? succ_y_outside : (g.lane < 31 ? y_from_above : read_slot<ST>(b_y, hi));
#pragma unroll
            for (int j = 0; j < E; ++j) {
                op.c[j] = (j == 0) ? c_pred : craw[j - 1];
                op.ysh[j] = (j == E - 1) ? y_succ : yraw[j + 1];
            }
        } else {     // predecessor = slot above, successor = slot below
            const float c_from_above = __shfl_down_sync(0xffffffffu, craw[0], 1);
            const float y_from_below = __shfl_up_sync(0xffffffffu, yraw[E - 1], 1);
            const float c_pred = !hi_ok ? pred_c_outside : (g.lane < 31 ? c_from_above : edge_coeff<ST>(b_c, hi, logc));
            const float y_succ = !lo_ok ? succ_y_outside : (g.lane > 0 ? y_from_below : read_slot<ST>(b_y, lo));
#pragma unroll
            for (int j = 0; j < E; ++j) {
                op.c[j] = (j == E - 1) ? c_pred : craw[j + 1];
                op.ysh[j] = (j == 0) ? y_succ : yraw[j - 1];
            }
        }
    }
    if constexpr (BWD) {
        // gradient with respect to the logarithm: d_c * c, folded into the shifted outputs that
        // d_c = d_x * y_shifted is formed from
        if (logc) {
#pragma unroll
            for (int j = 0; j < E; ++j) op.ysh[j] *= craw[j];
        }
    }
    // Slots past the end of the row are identity elements (x = 0 already, c = 1).
    if (PATCH && valid < g.tpr * E) {
#pragma unroll
        for (int j = 0; j < E; ++j)
            if (ra + j >= valid) op.c[j] = 1.0f;
    }
    // Nothing precedes the first element of a row: its coefficient is defined away, as in the
    // reference kernels that start with y[s] = x[s] (linrec/impl/cuda/linrec_ref.cuh:63).
    if (zero_first) op.c[ASC ? 0 : E - 1] = 0.0f;
}

// ---- scan state carried between the phases of one tile -----------------------------------------
struct ThreadScan {
    Pair agg;    // the thread's own E slots
    Pair excl;   // same-row lanes of this warp that precede the thread (identity if none)
};

// Phase 1: thread aggregate, then a segmented Kogge-Stone scan across the warp in scan order.
// The scan-last lane of every warp leaves the warp's inclusive value in wagg[ws].
template <int E, int NT, bool BWD, bool ASC>
__device__ __forceinline__ ThreadScan scan_thread_and_warp(const Operands<E, BWD>& op,
                                                           const Geometry& g, Pair* wagg)
{
    ThreadScan ts;
    Pair a = pair_identity();
#pragma unroll
    for (int jj = 0; jj < E; ++jj) {
        const int j = ASC ? jj : E - 1 - jj;
        a.y = fmaf(a.y, op.c[j], op.x[j]);
        a.p = a.p * op.c[j];
    }
    ts.agg = a;
    Pair inc = a;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int src = ASC ? g.lane - d : g.lane + d;
        Pair far;
        far.y = __shfl_sync(0xffffffffu, inc.y, src);
        far.p = __shfl_sync(0xffffffffu, inc.p, src);
        if (g.ls >= d && g.k >= d) inc = combine(far, inc);
    }
    Pair ex;
    {
        const int src = ASC ? g.lane - 1 : g.lane + 1;
        ex.y = __shfl_sync(0xffffffffu, inc.y, src);
        ex.p = __shfl_sync(0xffffffffu, inc.p, src);
    }
    ts.excl = g.has_excl ? ex : pair_identity();
    if (g.ls == 31) wagg[g.ws] = inc;
    return ts;
}

// Phase 2a (after a block barrier): what the earlier warps contribute to this thread's row.
// All warp aggregates are read up front (independent broadcast loads) and folded under a
// predicate, so the dependent chain is NW fused multiply-adds and not NW shared-memory round trips.
template <int NW>
__device__ __forceinline__ Pair cross_warp_prefix(const Geometry& g, const Pair* wagg)
{
    Pair a[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) a[w] = wagg[w];
    Pair wp = pair_identity();
#pragma unroll
    for (int w = 0; w < NW - 1; ++w)
        if (w >= g.start_warp && w < g.ws) wp = combine(wp, a[w]);
    return wp;
}

// Ordered reduction across a warp: lane 0 ends with v[31] o v[30] o ... o v[0]
// (higher lanes are FARTHER back in scan order).
__device__ __forceinline__ Pair warp_reduce_far_to_near(Pair v, int lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        Pair far;
        far.y = __shfl_down_sync(0xffffffffu, v.y, d);
        far.p = __shfl_down_sync(0xffffffffu, v.p, d);
        if (lane + d < 32) v = combine(far, v);
    }
    return v;
}

// Descriptor access: one 128-bit relaxed load / store at GPU scope.
// The returned word has its status reduced to the state (0, 1, 2) as seen from `epoch`.
__device__ __forceinline__ uint4 desc_load(const TileDesc* d, uint32_t epoch)
{
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(d)
                 : "memory");
    v.z = ((v.z >> 2) == epoch) ? (v.z & 3u) : 0u;
    return v;
}

// Publishes a tile's aggregate (status 1) or inclusive value (status 2); one lane calls this.
__device__ __forceinline__ void publish(TileDesc* d, Pair v, uint32_t state, uint32_t epoch)
{
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(d), "r"(__float_as_uint(v.y)),
                 "r"(__float_as_uint(v.p)), "r"((epoch << 2) | state), "r"(0u)
                 : "memory");
}

// Launch epilogue, called by one thread of every CTA after the CTA's last access to the workspace:
// the CTA that finishes last makes the workspace ready for the next launch.
__device__ __forceinline__ bool finish_launch(uint32_t* header, uint32_t epoch)
{
    __threadfence();
    const uint32_t done = atomicAdd(header + 3, 1u);
    if (done == gridDim.x - 1) {
        header[0] = 0u;
        header[3] = 0u;
        header[2] = (epoch + 1u) & 0x3fffffffu;
        return true;
    }
    return false;
}

// End of a scan kernel (one thread per CTA): count this CTA as done; in a launch that takes part in
// a peer exchange the CTA that was last tells all ranks that this rank's records are complete.
__device__ __forceinline__ void finish_scan(const ScanParams& p, uint32_t epoch)
{
    if (finish_launch(p.header, epoch) && p.px_epoch != 0u) publish_records(p.px, p.px_epoch);
}

__device__ __forceinline__ uint32_t read_epoch(const uint32_t* header)
{
    return *reinterpret_cast<const volatile uint32_t*>(header + 2);
}

__device__ __forceinline__ Pair desc_pair(const uint4& v) { return Pair{__uint_as_float(v.x), __uint_as_float(v.y)}; }

// Phase 2b, chain mode, run by ONE warp: decoupled look-back over the predecessor tiles of the
// same row.  Tile (row r, scan piece q) has ticket q*numseq + r, so its predecessor is `numseq`
// tickets back.  Returns (on every lane) the exclusive prefix of this tile.  One step of the walk
// looks at 32 predecessors, one per lane (nearest = lane 0), and folds them up to the nearest one
// that holds an inclusive value.  (Requesting the descriptors of several windows per round trip was
// measured and did not pay: where the walk is long, the tiles it waits for are still being scanned.)
// Each poll is bounded by p.wait_budget clock ticks; on expiry the status word is flagged and the
// missing predecessor is treated as an inclusive identity so that the walk terminates.
__device__ __forceinline__ Pair lookback(const ScanParams& p, uint32_t epoch, long long ticket, int q, int lane)
{
    Pair acc = pair_identity();
    int j0 = 1;
    while (true) {
        const int pq = q - j0 - lane;
        Pair v = pair_identity();
        uint32_t st = 2u;
        if (pq >= 0) {
            const TileDesc* d = p.desc + (ticket - (long long)(j0 + lane) * p.numseq);
            uint4 w = desc_load(d, epoch);
            if (w.z == 0u) {
                const long long t0 = clock64();
                unsigned ns = 32;
                while ((w = desc_load(d, epoch)).z == 0u) {
                    if (clock64() - t0 > p.wait_budget) break;
                    __nanosleep(ns);
                    if (ns < 1024) ns <<= 1;
                }
            }
            st = w.z;
            if (st == 0u) {
                atomicOr(p.header + 1, kStatusLookbackTimeout);
                st = 2u;   // give up: pretend an inclusive identity so that the walk ends
            } else {
                v = desc_pair(w);
            }
        }
        const uint32_t ball = __ballot_sync(0xffffffffu, st == 2u);
        const int first = ball ? (__ffs(ball) - 1) : 31;   // nearest predecessor holding an inclusive value
        if (lane > first) v = pair_identity();
        const Pair win = warp_reduce_far_to_near(v, lane);
        Pair w0;
        w0.y = __shfl_sync(0xffffffffu, win.y, 0);
        w0.p = __shfl_sync(0xffffffffu, win.p, 0);
        acc = combine(w0, acc);   // this window lies farther back than what was gathered so far
        if (ball) break;
        j0 += 32;
    }
    return acc;
}

// Phase 3: rerun the recurrence through the thread's slots from the true carry-in, which makes
// every output the result of the same fused multiply-adds a sequential walk would perform from
// that carry.
template <int E, bool BWD, bool ASC>
__device__ __forceinline__ void apply_carry(const Operands<E, BWD>& op, float carry_in,
                                            float (&o0)[E], float (&o1)[BWD ? E : 1])
{
    float v = carry_in;
#pragma unroll
    for (int jj = 0; jj < E; ++jj) {
        const int j = ASC ? jj : E - 1 - jj;
        v = fmaf(v, op.c[j], op.x[j]);
        o0[j] = v;
        if (BWD) o1[j] = v * op.ysh[j];
    }
}

}  // namespace linrec
