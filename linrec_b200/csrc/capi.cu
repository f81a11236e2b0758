// Host side of the library: argument checks, regime selection, tensor-map construction,
// workspace preparation and kernel launches, behind the C ABI of include/linrec_b200.h.
//
// Replaces the reference's host launchers and compile-time dispatch
// (linrec/impl/cuda/linrec_pipe.cu:16-212, linrec_tile.cu:17-215, linrec_ref.cu:11-95,
// dispatch.h:53-108) and the selection procedure of eval/tune.py:58-134, which there only prints
// tables: here a closed-form selector picks the variant from (rows, length, dtype, alignment).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/linrec_b200.h"
#include "variants.h"
#include "shard_kernels.cuh"

namespace {

using linrec::ScanParams;
using linrec::TileDesc;

std::atomic<uint64_t> g_launches{0};

// Text of the last CUDA error a call of this thread ran into (what LINREC_ERR_CUDA stands for).
thread_local char g_last_cuda_error[192] = "";
void note_cuda_error(const char* where, const char* what)
{
    snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", where, what ? what : "unknown error");
}
// Result of a kernel launch: reads (and clears) the runtime's last error.
int launch_result(const char* where)
{
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return LINREC_OK;
    note_cuda_error(where, cudaGetErrorString(e));
    return LINREC_ERR_CUDA;
}

// Launch with (or without) the programmatic-stream-serialization attribute: the kernels that take it
// call griddepcontrol.wait before their first access to global memory (ptx.cuh).
template <typename... KArgs, typename... Args>
void launch_kernel(void (*fn)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream, bool pdl, Args&&... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = pdl ? attr : nullptr;
    cfg.numAttrs = pdl ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, fn, std::forward<Args>(args)...);   // the caller reads cudaGetLastError
}

// ---- options -------------------------------------------------------------------------------------
// Compile-time configuration names (the counterpart of CONFIG_NAMES, linrec/impl/cuda/linrec.h:8).
const char* const kConfigNames[] = {"kElemsPerThread", "kThreadsPerBlock", "kStages", "kOutBuffers", "memcode"};
constexpr int kNumConfigNames = 5;
// memcode: 0 = plain coalesced loads/stores staged through shared memory (any alignment),
//          1 = tiled bulk-tensor copies (TMA) through an mbarrier ring (rows of whole 128-byte lines),
//          2 = 16-byte cp.async through a two-slot ring (16-byte aligned rows of whole 16-byte chunks),
//          3 = 4-byte cp.async through a two-slot ring (4-byte aligned rows of whole 4-byte words),
//          4 = one CTA per row with aligned 16-byte accesses (any length and offset; chosen by itself for
//              rows that 1 and 2 cannot take when there are several rows per SM; not in the variant
//              list: it has no tile parameters to pin).

struct Options {
    int E = -1, NT = -1, S = -1, OB = -1, memcode = -1;
    int wait_budget_ms = 2000;   // budget of every device-side wait
    int ctas_per_sm = 0;         // 0 = as many as fit
    int first_ticket = 0;        // diagnostics only: tickets start here instead of 0
    int lazy = -1;               // -1 = selector decides, 0/1 = one-ticket-at-a-time mode off/on (one ring slot only)
    int l2_promotion = 3;        // tensor-map L2 promotion: 0 none, 1 64 B, 2 128 B, 3 256 B
    int p2p_phase = 0;           // peer-exchange calls: 0 = scan and fix-up, 1 = scan only, 2 = fix-up only
    int LC = -1;                 // scan along the middle axis: sequence positions per chunk
    int K = -1;                  // scan along the middle axis: chunks per job (0 = whole column)
    int logc = 0;                // 1: the coefficient tensor holds logarithms
    int super_chunks = -1;       // few very long rows: -1 = selector decides, 0/1 = off, N (a power of two) = cut every row into N
    int fixup_threads = 128;     // measurements only: threads per CTA of the fix-up kernel (128 or 256; 128 measured 1-10 % faster)
    int pdl = 1;                 // programmatic dependent launch: the kernel may begin (up to its first access to
                                 // global memory) while the kernel before it in the stream is draining
    int fixed_first = 0;         // measurements only: chained rows also start from fixed round-robin tickets
    int peer_wait_budget_ms = 30000;   // budget of a wait for ANOTHER RANK (its records, its acknowledgements)
};

int parse_options(const linrec_opts* o, Options& out)
{
    if (!o || o->n_opts == 0) return LINREC_OK;
    if (o->n_opts < 0 || !o->names || !o->values) return LINREC_ERR_INVALID_ARG;
    for (int i = 0; i < o->n_opts; ++i) {
        const char* n = o->names[i];
        const int v = o->values[i];
        if (!n) return LINREC_ERR_INVALID_ARG;
        if (!strcmp(n, "kElemsPerThread")) out.E = v;
        else if (!strcmp(n, "kThreadsPerBlock")) out.NT = v;
        else if (!strcmp(n, "kStages")) out.S = v;
        else if (!strcmp(n, "kOutBuffers")) out.OB = v;
        else if (!strcmp(n, "kRowsPerChunk")) out.LC = v;
        else if (!strcmp(n, "kChunksPerJob")) out.K = v;
        else if (!strcmp(n, "logCoeffs")) out.logc = v != 0;
        else if (!strcmp(n, "memcode")) out.memcode = v;
        else if (!strcmp(n, "waitBudgetMs")) out.wait_budget_ms = v;
        else if (!strcmp(n, "ctasPerSm")) out.ctas_per_sm = v;
        else if (!strcmp(n, "firstTicket")) out.first_ticket = v;
        else if (!strcmp(n, "p2pPhase")) out.p2p_phase = v;
        else if (!strcmp(n, "lazyTickets")) out.lazy = v;
        else if (!strcmp(n, "l2Promotion")) out.l2_promotion = v;
        else if (!strcmp(n, "fixedFirstTickets")) out.fixed_first = v != 0;
        else if (!strcmp(n, "superChunks")) out.super_chunks = v;
        else if (!strcmp(n, "programmaticLaunch")) out.pdl = v != 0;
        else if (!strcmp(n, "fixupThreads")) out.fixup_threads = v;
        else if (!strcmp(n, "peerWaitBudgetMs")) out.peer_wait_budget_ms = v;
        else return LINREC_ERR_NOT_IMPLEMENTED;
    }
    return LINREC_OK;
}

using namespace linrec_variants;

const std::vector<TmaVariant>& tma_variants()
{
    static const std::vector<TmaVariant> v = [] {
        std::vector<TmaVariant> t;
        add_tma_variants_0(t);
        add_tma_variants_1(t);
        add_tma_variants_2(t);
        return t;
    }();
    return v;
}

const std::vector<GenericVariant>& generic_variants()
{
    static const std::vector<GenericVariant> v = {
        make_generic_variant<16, 128>(),
        make_generic_variant<8, 128>(),
    };
    return v;
}

// 16-byte cp.async loader, two ring slots: aligned rows whose length is not a multiple of 128 bytes
const std::vector<GenericVariant>& async_variants()
{
    static const std::vector<GenericVariant> v = [] {
        std::vector<GenericVariant> t;
        add_async_variants(t);
        return t;
    }();
    return v;
}

// 4-byte cp.async loader: rows of whole 4-byte words at 4-byte aligned addresses (any fp32 row)
const std::vector<GenericVariant>& word_variants()
{
    static const std::vector<GenericVariant> v = [] {
        std::vector<GenericVariant> t;
        add_word_variants(t);
        return t;
    }();
    return v;
}

// ---- per-device facts and per-kernel launch facts ------------------------------------------------
struct DeviceInfo {
    int sm_count = 0;
    int clock_khz = 0;
    int max_smem_optin = 0;
};

std::mutex g_mutex;
std::unordered_map<int, DeviceInfo> g_devices;

struct KernelKey {
    const void* fn;
    int device;
    bool operator==(const KernelKey& o) const { return fn == o.fn && device == o.device; }
};
struct KernelKeyHash {
    size_t operator()(const KernelKey& k) const { return std::hash<const void*>()(k.fn) ^ (size_t)k.device * 0x9e3779b97f4a7c15ull; }
};
std::unordered_map<KernelKey, int, KernelKeyHash> g_occupancy;   // resident CTAs per SM

int device_info(DeviceInfo& out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return LINREC_ERR_CUDA;
    // Tensor maps are encoded through a driver entry point, which needs the device's primary context
    // to be current in the calling thread.  The runtime binds it lazily, and a thread that has only
    // made calls that do not need one (an autograd worker with warm caches) has none yet.
    // cudaSetDevice on the device that is already selected does exactly that binding (it initialises
    // the primary context if need be and makes it current) and allocates or frees nothing.
    thread_local int bound_device = -1;
    if (bound_device != dev) {
        if (cudaSetDevice(dev) != cudaSuccess) {
            note_cuda_error("cudaSetDevice", "could not bind the device context in this thread");
            cudaGetLastError();
            return LINREC_ERR_CUDA;
        }
        bound_device = dev;
    }
    // the calling thread's own copy first: no lock on the path every launch takes
    thread_local int known_device = -1;
    thread_local DeviceInfo known;
    if (known_device == dev) {
        out = known;
        return LINREC_OK;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_devices.find(dev);
    if (it == g_devices.end()) {
        DeviceInfo d;
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return LINREC_ERR_CUDA;
        if (cudaDeviceGetAttribute(&d.clock_khz, cudaDevAttrClockRate, dev) != cudaSuccess) return LINREC_ERR_CUDA;
        if (cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return LINREC_ERR_CUDA;
        it = g_devices.emplace(dev, d).first;
    }
    out = it->second;
    known = it->second;
    known_device = dev;
    return LINREC_OK;
}

// Resident CTAs per SM for a kernel with `smem` bytes of dynamic shared memory; the first query on
// a device also raises the kernel's dynamic shared-memory limit.
int occupancy(const void* fn, int threads, size_t smem, int& out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return LINREC_ERR_CUDA;
    const KernelKey key{fn, dev};
    // the calling thread's last few answers first: no lock on the path every launch takes
    struct Recent {
        KernelKey key;
        int n;
    };
    thread_local Recent recent[8] = {};
    thread_local int recent_next = 0;
    for (const Recent& r : recent)
        if (r.n > 0 && r.key == key) {
            out = r.n;
            return LINREC_OK;
        }
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_occupancy.find(key);
    if (it == g_occupancy.end()) {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) {
                cudaGetLastError();
                note_cuda_error("cudaFuncSetAttribute(MaxDynamicSharedMemorySize)", cudaGetErrorString(e));
                return LINREC_ERR_CUDA;
            }
        }
        int n = 0;
        const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, smem);
        if (e != cudaSuccess) {
            cudaGetLastError();
            note_cuda_error("cudaOccupancyMaxActiveBlocksPerMultiprocessor", cudaGetErrorString(e));
            return LINREC_ERR_CUDA;
        }
        if (n <= 0) note_cuda_error("occupancy", "the kernel does not fit an SM with this much shared memory");
        it = g_occupancy.emplace(key, n).first;
    }
    out = it->second;
    if (out > 0) {
        recent[recent_next] = Recent{key, out};
        recent_next = (recent_next + 1) % 8;
    }
    return out > 0 ? LINREC_OK : LINREC_ERR_CUDA;
}

// ---- tensor maps ---------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Rank-3 view (elements of a 128-byte line, lines of a row, rows) of a row-major matrix with a
// 128-byte swizzle; box = (one line, `box_lines`, `box_rows`).
int make_map(CUtensorMap* map, const void* ptr, int dtype, int64_t numseq, int64_t seqlen,
             int64_t row_stride, int box_lines, int box_rows, int l2_promotion)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        note_cuda_error("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled not found");
        return LINREC_ERR_CUDA;
    }
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    const cuuint64_t epl = 128 / sz;
    const cuuint64_t dims[3] = {epl, (cuuint64_t)(seqlen / (int64_t)epl), (cuuint64_t)numseq};
    const cuuint64_t strides[2] = {128, (cuuint64_t)row_stride * (cuuint64_t)sz};
    const cuuint32_t box[3] = {(cuuint32_t)epl, (cuuint32_t)box_lines, (cuuint32_t)box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, dtype == LINREC_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == LINREC_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B,
                           l2_promotion == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                           : l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                           : l2_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof(msg), "driver error %d", (int)r);
        note_cuda_error("cuTensorMapEncodeTiled", msg);
        return LINREC_ERR_CUDA;
    }
    return LINREC_OK;
}

// Encoding a tensor map costs about a microsecond and a launch needs five; a training loop calls with
// the same buffers and shapes over and over.  Each host thread therefore keeps the last few maps it
// encoded (no lock; a map depends on nothing but the arguments that make up the key).
struct MapKey {
    const void* ptr;
    int64_t numseq, seqlen, row_stride;
    int dtype, box_lines, box_rows, l2;
    bool operator==(const MapKey& o) const
    {
        return ptr == o.ptr && numseq == o.numseq && seqlen == o.seqlen && row_stride == o.row_stride && dtype == o.dtype &&
               box_lines == o.box_lines && box_rows == o.box_rows && l2 == o.l2;
    }
};
int cached_map(CUtensorMap* map, const void* ptr, int dtype, int64_t numseq, int64_t seqlen, int64_t row_stride,
               int box_lines, int box_rows, int l2_promotion)
{
    constexpr int kSlots = 16;
    struct Slot {
        MapKey key;
        CUtensorMap map;
        bool used;
    };
    thread_local Slot slots[kSlots] = {};
    thread_local int next = 0;
    const MapKey key{ptr, numseq, seqlen, row_stride, dtype, box_lines, box_rows, l2_promotion};
    for (int i = 0; i < kSlots; ++i)
        if (slots[i].used && slots[i].key == key) {
            *map = slots[i].map;
            return LINREC_OK;
        }
    const int rc = make_map(map, ptr, dtype, numseq, seqlen, row_stride, box_lines, box_rows, l2_promotion);
    if (rc != LINREC_OK) return rc;
    Slot& s = slots[next];
    next = (next + 1) % kSlots;
    s.key = key;
    s.map = *map;
    s.used = true;
    return LINREC_OK;
}

// ---- planning ------------------------------------------------------------------------------------
struct Plan {
    bool tma = false;
    bool async_copy = false;   // cp.async ring, 16-byte (memcode 2) or 4-byte (memcode 3) chunks
    const TmaVariant* tv = nullptr;
    const GenericVariant* gv = nullptr;
    int E = 0, NT = 0, T = 0;
    int chain = 0, slots_per_row = 0, rows_per_tile = 1, chunks_per_row = 1;
    long long ntiles = 0;
    bool lazy_default = false;
    int memcode = 0;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

bool tma_eligible(int dtype, int64_t numseq, int64_t seqlen, int64_t row_stride, const void* const* ptrs, int nptrs)
{
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    if ((seqlen * sz) % 128 != 0) return false;
    if ((row_stride * sz) % 16 != 0) return false;
    if (numseq > 0x7fffffffLL || seqlen / (128 / sz) > 0x7fffffffLL) return false;
    if ((uint64_t)row_stride * sz >= (1ull << 40)) return false;
    for (int i = 0; i < nptrs; ++i)
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return false;
    return true;
}

// 16-byte global accesses outside the bulk-copy kernel: aligned rows of whole 16-byte chunks
bool vec_eligible(int dtype, int64_t seqlen, int64_t row_stride, const void* const* ptrs, int nptrs)
{
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    if ((row_stride * sz) % 16 != 0 || (seqlen * sz) % 16 != 0) return false;
    for (int i = 0; i < nptrs; ++i)
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return false;
    return true;
}

// 4-byte asynchronous copies: rows of whole 4-byte words at 4-byte aligned addresses
bool word_eligible(int dtype, int64_t seqlen, int64_t row_stride, const void* const* ptrs, int nptrs)
{
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    if ((row_stride * sz) % 4 != 0 || (seqlen * sz) % 4 != 0) return false;
    for (int i = 0; i < nptrs; ++i)
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % 4 != 0) return false;
    return true;
}

// Tile-shape bookkeeping shared by both loaders.
void shape_plan(Plan& pl, int dtype, int64_t numseq, int64_t seqlen)
{
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    const int64_t lp = pl.tma ? seqlen : round_up(seqlen, pl.E);
    if (lp > pl.T) {
        pl.chain = 1;
        pl.chunks_per_row = (int)ceil_div(seqlen, pl.T);
        pl.rows_per_tile = 1;
        pl.slots_per_row = pl.T;
        pl.ntiles = numseq * pl.chunks_per_row;
    } else {
        pl.chain = 0;
        pl.chunks_per_row = 1;
        pl.slots_per_row = (int)lp;
        int64_t r = pl.T / lp;
        if (pl.tma && r > 256) r = 256;          // box dimensions are limited to 256
        if (r > numseq) r = numseq;
        (void)sz;
        pl.rows_per_tile = (int)r;
        pl.ntiles = ceil_div(numseq, r);
    }
}

// The regime selector.  `kind` TILE refuses rows that do not fit one tile, as the reference's
// tile operator does (linrec/impl/cuda/linrec_tile.cu:60).
int make_plan(Plan& pl, int kind, bool bwd, int dtype, int64_t numseq, int64_t seqlen, int64_t row_stride,
              const void* const* ptrs, int nptrs, const Options& opt, int max_smem, int sm_count)
{
    const bool can_tma = tma_eligible(dtype, numseq, seqlen, row_stride, ptrs, nptrs);
    const bool can_vec = vec_eligible(dtype, seqlen, row_stride, ptrs, nptrs);
    const bool can_word = word_eligible(dtype, seqlen, row_stride, ptrs, nptrs);
    int memcode = opt.memcode;
    if (memcode < 0) memcode = can_tma ? 1 : (can_vec ? 2 : (can_word ? 3 : 0));
    if (memcode < 0 || memcode > 3) return LINREC_ERR_NOT_IMPLEMENTED;
    if (memcode == 1 && !can_tma) return LINREC_ERR_UNALIGNED;
    if (memcode == 2 && !can_vec) return LINREC_ERR_UNALIGNED;
    if (memcode == 3 && !can_word) return LINREC_ERR_UNALIGNED;
    pl.tma = memcode == 1;
    pl.async_copy = memcode == 2 || memcode == 3;
    pl.memcode = memcode;
    const int di = dtype == LINREC_DTYPE_F32 ? 0 : (dtype == LINREC_DTYPE_BF16 ? 1 : 2);
    if (pl.tma) {
        // Defaults of the selector (measured on B200, see the sweep of the standalone harness):
        // forward: 512 threads x 16 elements, two ring slots; backward: 128 x 16, two ring slots
        // (its five arrays per tile leave room for three such CTAs per SM).  The tile family needs
        // the whole row in one tile and therefore takes the smallest tile that holds the row.
        int E = opt.E, NT = opt.NT, S = opt.S, OB = opt.OB;
        const bool pinned = !(E < 0 && NT < 0 && S < 0 && OB < 0);
        if (!pinned && kind != LINREC_KIND_TILE) {
            const int sz = di == 0 ? 4 : 2;
            // rows shorter than the small tile never chain; with few long rows the predecessor of a
            // tile is often still in flight, and fewer, larger CTAs do better
            const bool short_rows = seqlen <= 2048;
            const bool few_rows = !short_rows && numseq < 4LL * sm_count;
            // a handful of very long rows: consecutive tickets are consecutive pieces of the same row,
            // so CTAs hold one ticket at a time (see the kernel's "lazy" mode)
            const bool handful = !short_rows && seqlen > 8192 && numseq < 32;
            pl.lazy_default = handful;
            auto padded = [&](int64_t tile) { return ceil_div(seqlen, tile) * tile; };   // slots a row takes in tiles of this size
            if (handful) {
                E = 16; NT = 512; S = 1; OB = 1;
            } else if (sz == 4) {
                // backward: one ring slot and more resident CTAs beat a deeper ring (five arrays per
                // tile); rows up to 8192 take the 8192-element tile and never chain
                // (a small forward problem of rows that fit the 4096-element tile: twice as many tiles
                // balance better over the SMs -- (512, 4096): 10.6 instead of 12.5 us per launch)
                const bool small = seqlen <= 4096 && numseq * seqlen < 4LL * sm_count * 8192;
                if (!bwd) {
                    E = 16; NT = small ? 256 : 512; S = 2; OB = 1;
                    // chained rows whose last 8192-element piece is mostly empty: a nearly empty tile costs
                    // almost what a full one does, so take the tile that pads the row least
                    // ((4096, 65568): 6094 -> 6450 GB/s, (26800, 10016): < 6000 -> 6500)
                    if (seqlen > 8192 && !few_rows && padded(8192) * 100 > std::min(padded(4096), padded(2048)) * 101) {
                        if (padded(4096) * 100 <= padded(2048) * 102) { NT = 256; S = 2; }
                        else                                          { NT = 128; S = 3; }
                    }
                }
                else if (seqlen <= 8192 || few_rows) { E = 16; NT = 512; S = 1; OB = 1; }
                else                               { E = 16; NT = 128; S = 1; OB = 1; }
            } else {
                // 2-byte storage moves half the bytes per element, so instruction issue starts to
                // matter: 32 elements per thread halve the shuffle and barrier cost per element
                // Few long rows: with two or more CTAs per SM there are more tiles being worked on than
                // there are rows, so a tile's predecessor is usually still in flight and the look-back
                // waits; one CTA per SM with a 16384-element tile (the bytes of an 8192-element fp32
                // tile) keeps the predecessor a whole round back.
                if (short_rows)     { E = 16; NT = 128; S = bwd ? 2 : 3; OB = 1; }
                else if (few_rows)  { E = 32; NT = 512; S = bwd ? 1 : 2; OB = 1; }
                else if (!bwd)      { E = 32; NT = (seqlen > 8192 && padded(8192) * 100 > padded(4096) * 101) ? 128 : 256; S = 2; OB = 1; }
                else                { E = 32; NT = 128; S = 2; OB = 1; }
            }
        }
        const TmaVariant* best = nullptr;
        for (const TmaVariant& v : tma_variants()) {
            if (!((E < 0 || v.E == E) && (NT < 0 || v.NT == NT) && (S < 0 || v.S == S) && (OB < 0 || v.OB == OB))) continue;
            if (v.smem[di][bwd] > (size_t)max_smem) continue;
            if ((size_t)v.E * v.NT * (di == 0 ? 4 : 2) > 256 * 128) continue;   // a copy box holds at most 256 lines of 128 bytes
            if (!pinned && kind == LINREC_KIND_TILE) {
                // smallest tile that holds the row; among equals the deeper ring
                if (v.E * v.NT < seqlen) continue;
                if (!best || v.E * v.NT < best->E * best->NT || (v.E * v.NT == best->E * best->NT && v.S > best->S)) best = &v;
            } else {
                best = &v;
                break;
            }
        }
        if (!best) {
            if (!pinned && kind == LINREC_KIND_TILE) return LINREC_ERR_TOO_LONG;
            return LINREC_ERR_NOT_IMPLEMENTED;
        }
        pl.tv = best;
        pl.E = pl.tv->E; pl.NT = pl.tv->NT;
    } else if (pl.async_copy) {
        if (opt.OB > 0) return LINREC_ERR_NOT_IMPLEMENTED;
        const bool pinned = !(opt.E < 0 && opt.NT < 0 && opt.S < 0);
        int E = opt.E, NT = opt.NT, S = opt.S;
        if (!pinned && kind != LINREC_KIND_TILE) {
            // Many rows: the small tile and many resident CTAs (4-byte rows that fit it: the 4096-element
            // tile, three CTAs per SM, measured faster than six small ones).  Few long rows: consecutive tickets are
            // pieces of the same row and wait for each other, so larger tiles; a handful of very long
            // rows: the largest tile, one ticket at a time.
            const bool few_rows = seqlen > 2048 && numseq < 4LL * sm_count;
            const bool handful = seqlen > 8192 && numseq < 32;
            pl.lazy_default = handful;
            S = 2;
            if (handful)            { E = 16; NT = 512; }
            else if (memcode == 3)  { E = 16; NT = 128; }   // word copies: the small tile won every sweep
            else if (few_rows)      { E = 32; NT = 128; }
            else if (di == 0 && seqlen <= 4096) { E = 16; NT = 256; }   // 4-byte rows that fit the 4096-element tile
            else                    { E = 16; NT = 128; }
        }
        for (const GenericVariant& v : (memcode == 2 ? async_variants() : word_variants())) {
            if (!((E < 0 || v.E == E) && (NT < 0 || v.NT == NT) && (S < 0 || v.S == S))) continue;
            if (v.smem[di][bwd] > (size_t)max_smem) continue;
            if (!pinned && kind == LINREC_KIND_TILE) {
                // smallest tile that holds the (padded) row
                if (v.E * v.NT < round_up(seqlen, v.E)) continue;
                if (!pl.gv || v.E * v.NT < pl.gv->E * pl.gv->NT) pl.gv = &v;
            } else {
                pl.gv = &v;
                break;
            }
        }
        if (!pl.gv) return (!pinned && kind == LINREC_KIND_TILE) ? LINREC_ERR_TOO_LONG : LINREC_ERR_NOT_IMPLEMENTED;
        pl.E = pl.gv->E; pl.NT = pl.gv->NT;
    } else {
        if (opt.S > 1 || opt.OB > 0) return LINREC_ERR_NOT_IMPLEMENTED;
        for (const GenericVariant& v : generic_variants()) {
            if ((opt.E < 0 || v.E == opt.E) && (opt.NT < 0 || v.NT == opt.NT)) {
                pl.gv = &v;
                break;
            }
        }
        if (!pl.gv) return LINREC_ERR_NOT_IMPLEMENTED;
        pl.E = pl.gv->E; pl.NT = pl.gv->NT;
    }
    pl.T = pl.E * pl.NT;
    shape_plan(pl, dtype, numseq, seqlen);
    if (kind == LINREC_KIND_TILE && pl.chain) return LINREC_ERR_TOO_LONG;
    if (pl.ntiles >= 0x7ff00000LL) return LINREC_ERR_INVALID_ARG;   // tickets are 32-bit
    return LINREC_OK;
}

size_t workspace_need(const Plan& pl)
{
    size_t n = linrec::kHeaderBytes;
    if (pl.chain) n += (size_t)pl.ntiles * sizeof(TileDesc);
    return n;
}

int check_common(const void* const* ptrs, int nptrs, int64_t numseq, int64_t seqlen, int64_t row_stride, int dtype)
{
    if (dtype != LINREC_DTYPE_F32 && dtype != LINREC_DTYPE_BF16 && dtype != LINREC_DTYPE_F16 && dtype != LINREC_DTYPE_F64)
        return LINREC_ERR_NOT_IMPLEMENTED;
    if (numseq < 0 || seqlen < 0) return LINREC_ERR_INVALID_ARG;
    if (numseq == 0 || seqlen == 0) return LINREC_OK;
    if (row_stride < seqlen) return LINREC_ERR_INVALID_ARG;
    const int sz = dtype == LINREC_DTYPE_F64 ? 8 : dtype == LINREC_DTYPE_F32 ? 4 : 2;
    for (int i = 0; i < nptrs; ++i) {
        if (!ptrs[i]) return LINREC_ERR_INVALID_ARG;
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % sz != 0) return LINREC_ERR_INVALID_ARG;
    }
    return LINREC_OK;
}

// The one launcher behind forward, backward and the carry-emitting forward: ONE kernel launch.
int launch_scan_direct(int kind, bool bwd, const void* in0, const void* c, const void* yin, void* out0, void* out1,
                       float* carry_out, int carry_stride, int open_start, const void* exchange, uint32_t px_epoch, int64_t numseq, int64_t seqlen, int64_t row_stride,
                       int reverse, int dtype, const linrec_opts* opts, void* workspace, size_t workspace_bytes,
                       void* stream_, int super_chunks = 0)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const void* ptrs[5] = {in0, c, out0, bwd ? yin : in0, bwd ? out1 : out0};
    int rc = check_common(ptrs, 5, numseq, seqlen, row_stride, dtype);
    if (rc != LINREC_OK) return rc;
    if (kind != LINREC_KIND_REF && kind != LINREC_KIND_TILE && kind != LINREC_KIND_PIPE) return LINREC_ERR_INVALID_ARG;
    Options opt;
    rc = parse_options(opts, opt);
    if (rc != LINREC_OK) return rc;
    if (numseq == 0 || seqlen == 0) return LINREC_OK;

    DeviceInfo dev;
    rc = device_info(dev);
    if (rc != LINREC_OK) return rc;

    ScanParams p{};
    p.in0 = in0; p.c = c; p.yin = yin; p.out0 = out0; p.out1 = out1;
    p.numseq = numseq; p.seqlen = seqlen; p.row_stride = row_stride;
    p.carry_out = carry_out;
    p.carry_stride = carry_stride;
    p.open_start = open_start;
    p.super_chunks = super_chunks;
    p.px = static_cast<const linrec::PeerTable*>(exchange);
    p.px_epoch = exchange ? px_epoch : 0u;
    p.logc = opt.logc;
    // the carry records and fix-up kernels of sequence sharding work on plain coefficients
    if (opt.logc && (carry_out || exchange || open_start)) return LINREC_ERR_NOT_IMPLEMENTED;
    p.wait_budget = (long long)opt.wait_budget_ms * (long long)dev.clock_khz;
    p.peer_wait_budget = (long long)opt.peer_wait_budget_ms * (long long)dev.clock_khz;
    p.fixed_first = opt.fixed_first;
    const int di = dtype == LINREC_DTYPE_F32 ? 0 : (dtype == LINREC_DTYPE_BF16 ? 1 : 2);
    // the gradient scan runs against the direction of the forward pass
    const bool asc = bwd ? (reverse != 0) : (reverse == 0);

    // double precision (fp64 storage and arithmetic): the sequential operator, and for the tiled families
    // one kernel that gives every row to one CTA (no look-back, no workspace, no variants to pin)
    if (dtype == LINREC_DTYPE_F64 && (carry_out || exchange || open_start)) return LINREC_ERR_NOT_IMPLEMENTED;
    if (dtype == LINREC_DTYPE_F64 && kind != LINREC_KIND_REF) {
        if (opt.E >= 0 || opt.NT >= 0 || opt.S >= 0 || opt.OB >= 0 || opt.memcode >= 0) return LINREC_ERR_NOT_IMPLEMENTED;
        const unsigned blocks = (unsigned)std::min<int64_t>(numseq, (int64_t)dev.sm_count * 8);
        bool vec = row_stride % 2 == 0 && (asc || seqlen % 2 == 0);
        for (const void* q : ptrs) vec = vec && reinterpret_cast<uintptr_t>(q) % 16 == 0;
        auto launch = [&](auto kernel) { kernel<<<blocks, 256, 0, stream>>>(p); };
        auto pick = [&](auto bwd_c, auto asc_c) {
            constexpr bool B = decltype(bwd_c)::value, A = decltype(asc_c)::value;
            if (vec) { if (opt.logc) launch(linrec::linrec_row_f64_kernel<B, A, true, true>); else launch(linrec::linrec_row_f64_kernel<B, A, true, false>); }
            else     { if (opt.logc) launch(linrec::linrec_row_f64_kernel<B, A, false, true>); else launch(linrec::linrec_row_f64_kernel<B, A, false, false>); }
        };
        if (bwd) { if (asc) pick(std::true_type{}, std::true_type{}); else pick(std::true_type{}, std::false_type{}); }
        else     { if (asc) pick(std::false_type{}, std::true_type{}); else pick(std::false_type{}, std::false_type{}); }
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return launch_result("kernel launch");
    }
    // Rows that neither the bulk copies nor the 16-byte chunk copies can take (odd lengths, rows that
    // start off a 16-byte boundary): with enough rows to give every SM several, one CTA walks one row
    // with aligned 16-byte accesses (`memcode` 4; not a member of the variant list: it has no tile
    // parameters to pin).  (268167, 1001) fp32: 3.9 / 4.3 TB/s with the 4-byte copies.
    if (kind != LINREC_KIND_REF && dtype != LINREC_DTYPE_F64 && !carry_out && !exchange && !open_start &&
        (opt.memcode == 4 || (opt.memcode < 0 && opt.E < 0 && opt.NT < 0 && opt.S < 0 && opt.OB < 0))) {
        bool same_offset = true;
        for (const void* q : ptrs)
            same_offset = same_offset && reinterpret_cast<uintptr_t>(q) % 16 == reinterpret_cast<uintptr_t>(in0) % 16;
        const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
        same_offset = same_offset && (reinterpret_cast<uintptr_t>(in0) % sz == 0);
        const bool chunked = tma_eligible(dtype, numseq, seqlen, row_stride, ptrs, 5) || vec_eligible(dtype, seqlen, row_stride, ptrs, 5);
        // (short rows leave most of a CTA idle: where the 4-byte copies can take them they win below
        //  ~400 elements -- (1000000, 265) fp32: 3.8 against 1.9 TB/s with 128 threads; plain loads never do)
        const bool word_ok = word_eligible(dtype, seqlen, row_stride, ptrs, 5);
        const bool wanted = opt.memcode == 4 || (!chunked && numseq >= 4LL * dev.sm_count && seqlen >= (word_ok ? 384 : 48));
        if (opt.memcode == 4 && (!same_offset || (kind == LINREC_KIND_TILE && seqlen > 8192))) return LINREC_ERR_UNALIGNED;
        if (wanted && same_offset && !(kind == LINREC_KIND_TILE && seqlen > 8192)) {
            if (opt.E >= 0 || opt.NT >= 0 || opt.S >= 0 || opt.OB >= 0) return LINREC_ERR_NOT_IMPLEMENTED;
            // threads per CTA (x 8 elements = one tile): the smallest tile that holds the row, up to 2048 elements
            const int threads = seqlen > 1024 ? 256 : (seqlen > 512 ? 128 : 64);
            const unsigned blocks = (unsigned)std::min<int64_t>(numseq, (int64_t)dev.sm_count * std::min(2048 / threads, 24));
            auto launch = [&](auto kernel) { kernel<<<blocks, threads, 0, stream>>>(p); };
            auto pick = [&](auto st, auto bwd_c, auto asc_c) {
                using ST = decltype(st);
                constexpr bool B = decltype(bwd_c)::value, A = decltype(asc_c)::value;
                if (threads == 256)      launch(linrec::linrec_row_kernel<ST, 256, B, A>);
                else if (threads == 128) launch(linrec::linrec_row_kernel<ST, 128, B, A>);
                else                     launch(linrec::linrec_row_kernel<ST, 64, B, A>);
            };
            auto by_dir = [&](auto st) {
                if (bwd) { if (asc) pick(st, std::true_type{}, std::true_type{}); else pick(st, std::true_type{}, std::false_type{}); }
                else     { if (asc) pick(st, std::false_type{}, std::true_type{}); else pick(st, std::false_type{}, std::false_type{}); }
            };
            if (di == 0) by_dir(float{}); else if (di == 1) by_dir(__nv_bfloat16{}); else by_dir(__half{});
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return launch_result("kernel launch");
        }
    }
    if (kind == LINREC_KIND_REF) {
        if (carry_out) return LINREC_ERR_NOT_IMPLEMENTED;
        const int threads = dtype == LINREC_DTYPE_F64 ? 32 : 128;   // fp64 is the checker: spread few rows over many SMs
        const unsigned blocks = (unsigned)ceil_div(numseq, threads);
        if (dtype == LINREC_DTYPE_F64) {
            if (bwd) linrec::linrec_seq_f64_kernel<true><<<blocks, threads, 0, stream>>>(p, reverse);
            else     linrec::linrec_seq_f64_kernel<false><<<blocks, threads, 0, stream>>>(p, reverse);
        } else if (di == 0) {
            if (bwd) linrec::linrec_seq_kernel<float, true><<<blocks, threads, 0, stream>>>(p, reverse);
            else     linrec::linrec_seq_kernel<float, false><<<blocks, threads, 0, stream>>>(p, reverse);
        } else if (di == 1) {
            if (bwd) linrec::linrec_seq_kernel<__nv_bfloat16, true><<<blocks, threads, 0, stream>>>(p, reverse);
            else     linrec::linrec_seq_kernel<__nv_bfloat16, false><<<blocks, threads, 0, stream>>>(p, reverse);
        } else {
            if (bwd) linrec::linrec_seq_kernel<__half, true><<<blocks, threads, 0, stream>>>(p, reverse);
            else     linrec::linrec_seq_kernel<__half, false><<<blocks, threads, 0, stream>>>(p, reverse);
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return launch_result("kernel launch");
    }

    Plan pl;
    rc = make_plan(pl, kind, bwd, dtype, numseq, seqlen, row_stride, ptrs, 5, opt, dev.max_smem_optin, dev.sm_count);
    if (rc != LINREC_OK) return rc;

    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < workspace_need(pl))
        return LINREC_ERR_WORKSPACE;
    p.header = static_cast<uint32_t*>(workspace);
    p.desc = reinterpret_cast<TileDesc*>(static_cast<char*>(workspace) + linrec::kHeaderBytes);
    p.chain = pl.chain;
    p.slots_per_row = pl.slots_per_row;
    p.rows_per_tile = pl.rows_per_tile;
    p.chunks_per_row = pl.chunks_per_row;
    p.ntiles = pl.ntiles;

    const void* fn = pl.tma ? reinterpret_cast<const void*>(pl.tv->fn[di][bwd][asc])
                            : reinterpret_cast<const void*>(pl.gv->fn[di][bwd][asc]);
    const size_t smem = pl.tma ? pl.tv->smem[di][bwd] : pl.gv->smem[di][bwd];
    int occ = 0;
    rc = occupancy(fn, pl.NT, smem, occ);
    if (rc != LINREC_OK) return rc;
    if (opt.ctas_per_sm > 0 && opt.ctas_per_sm < occ) occ = opt.ctas_per_sm;
    long long grid = (long long)dev.sm_count * occ;
    if (grid > pl.ntiles) grid = pl.ntiles;

    // The workspace cleans up after every launch by itself (see scan_core.cuh): nothing to prepare.
    p.first_ticket = (uint32_t)opt.first_ticket;
    p.lazy = pl.chain && (pl.tma ? pl.tv->S == 1 : pl.async_copy) && (opt.lazy >= 0 ? opt.lazy != 0 : pl.lazy_default);
    p.vec = vec_eligible(dtype, seqlen, row_stride, ptrs, 5) ? 1 : 0;

    if (pl.tma) {
        CUtensorMap m[5];
        const int box_lines = pl.chain ? pl.T / (128 / (di == 0 ? 4 : 2)) : (int)(seqlen / (128 / (di == 0 ? 4 : 2)));
        const int box_rows = pl.chain ? 1 : pl.rows_per_tile;
        const void* src[5] = {in0, c, bwd ? yin : c, out0, bwd ? out1 : out0};
        for (int i = 0; i < 5; ++i) {
            rc = cached_map(&m[i], src[i], dtype, numseq, seqlen, row_stride, box_lines, box_rows, opt.l2_promotion);
            if (rc != LINREC_OK) return rc;
        }
        launch_kernel(pl.tv->fn[di][bwd][asc], (unsigned)grid, (unsigned)pl.NT, smem, stream, opt.pdl != 0, m[0], m[1], m[2], m[3],
                      m[4], p);
    } else {
        launch_kernel(pl.gv->fn[di][bwd][asc], (unsigned)grid, (unsigned)pl.NT, smem, stream, opt.pdl != 0, p);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return launch_result("kernel launch");
}

}  // namespace

// ---- sequence sharding -------------------------------------------------------------------------------
namespace {
// Does shard `shard` hold the element the scan starts from?
inline bool holds_scan_start(bool asc, int shard, int nshards) { return asc ? shard == 0 : shard == nshards - 1; }

template <typename ST, int NT>
int launch_fixup_t(bool bwd, bool asc, const linrec::FixupParams& fp, cudaStream_t stream, int sm_count)
{
    long long grid = fp.numseq < (long long)sm_count * 16 ? fp.numseq : (long long)sm_count * 16;
    // 16-byte accesses need aligned rows whose length is a multiple of the 8 elements a thread takes
    auto al = [](const void* q) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool vec = al(fp.out0) && al(fp.out1) && al(fp.in0) && al(fp.c) && al(fp.yin) && fp.seqlen % 8 == 0 &&
                     (fp.row_stride * (long long)sizeof(ST)) % 16 == 0;
    const unsigned g = (unsigned)grid;
#define LINREC_FIXUP(B, A, V) launch_kernel(linrec::linrec_fixup_kernel<ST, NT, B, A, V>, g, (unsigned)NT, 0, stream, true, fp)
    if (!bwd) {
        if (asc) { if (vec) LINREC_FIXUP(false, true, true); else LINREC_FIXUP(false, true, false); }
        else     { if (vec) LINREC_FIXUP(false, false, true); else LINREC_FIXUP(false, false, false); }
    } else {
        if (asc) { if (vec) LINREC_FIXUP(true, true, true); else LINREC_FIXUP(true, true, false); }
        else     { if (vec) LINREC_FIXUP(true, false, true); else LINREC_FIXUP(true, false, false); }
    }
#undef LINREC_FIXUP
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return launch_result("kernel launch");
}

int launch_fixup(bool bwd, const void* in0, void* out0, void* out1, const void* c, const void* yin, const float* carries,
                 const void* px, uint32_t px_epoch, uint32_t* status_word, int peer_wait_budget_ms, int64_t numseq,
                 int64_t seqlen, int64_t row_stride, int reverse, int dtype, int shard, int nshards, void* stream_,
                 int super_chunks = 0, int threads = 128)
{
    const void* ptrs[5] = {out0, c, in0, bwd ? out1 : out0, bwd ? yin : c};
    if (!carries && !px && numseq > 0 && seqlen > 0) return LINREC_ERR_INVALID_ARG;
    if (dtype == LINREC_DTYPE_F64) return LINREC_ERR_NOT_IMPLEMENTED;
    int rc = check_common(ptrs, 3, numseq, seqlen, row_stride, dtype);
    if (rc != LINREC_OK) return rc;
    if (bwd && (!out1 || !yin) && numseq > 0 && seqlen > 0) return LINREC_ERR_INVALID_ARG;
    if (nshards < 1 || shard < 0 || shard >= nshards) return LINREC_ERR_INVALID_ARG;
    if (numseq == 0 || seqlen == 0) return LINREC_OK;
    const bool asc = bwd ? (reverse != 0) : (reverse == 0);
    // nothing enters the shard that holds the scan start; with a peer exchange the kernel still runs
    // because it is the one that acknowledges the epoch to the other ranks
    if (holds_scan_start(asc, shard, nshards) && !bwd && !px && super_chunks <= 1) return LINREC_OK;
    DeviceInfo dev;
    rc = device_info(dev);
    if (rc != LINREC_OK) return rc;
    linrec::FixupParams fp{};
    fp.out0 = out0; fp.out1 = out1; fp.in0 = in0; fp.c = c; fp.yin = yin; fp.carries = carries;
    fp.numseq = numseq; fp.seqlen = seqlen; fp.row_stride = row_stride;
    fp.shard = shard; fp.nshards = nshards; fp.rec = bwd ? 4 : 2;
    fp.super_chunks = super_chunks;
    fp.px = static_cast<const linrec::PeerTable*>(px);
    fp.px_epoch = px ? px_epoch : 0u;
    fp.status = status_word;
    fp.wait_budget = (long long)peer_wait_budget_ms * (long long)dev.clock_khz;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (threads != 256)
        return dtype == LINREC_DTYPE_F32 ? launch_fixup_t<float, 128>(bwd, asc, fp, stream, dev.sm_count)
               : dtype == LINREC_DTYPE_BF16 ? launch_fixup_t<__nv_bfloat16, 128>(bwd, asc, fp, stream, dev.sm_count)
                                            : launch_fixup_t<__half, 128>(bwd, asc, fp, stream, dev.sm_count);
    return dtype == LINREC_DTYPE_F32 ? launch_fixup_t<float, 256>(bwd, asc, fp, stream, dev.sm_count)
           : dtype == LINREC_DTYPE_BF16 ? launch_fixup_t<__nv_bfloat16, 256>(bwd, asc, fp, stream, dev.sm_count)
                                        : launch_fixup_t<__half, 256>(bwd, asc, fp, stream, dev.sm_count);
}
}  // namespace


// ---- few, very long rows: super-chunks ------------------------------------------------------------------
// With fewer rows than CTAs, consecutive tiles of one row are in flight together and every tile waits
// for its predecessor: the chain of look-backs, not the memory system, sets the pace (about 3 TB/s).
// There every real row is cut into V consecutive super-chunks that are scanned as independent rows
// (all but the first one "open", exactly like the shards of a sequence that is split over GPUs), each
// leaving a record (P, Y[, edge elements]); a second, short kernel folds the records of the earlier
// super-chunks of the same row and computes the head of each super-chunk again from the true carry, as
// far as that carry lives (for decaying coefficients a few thousand elements at most; only coefficients
// that do not decay at all make it a full second pass).  The records live at the end of the workspace.
namespace {
constexpr int64_t kSuperChunkMaxRows = 128;       // regime: fewer rows than this ...
constexpr int64_t kSuperChunkMaxRowsBwd = 592;    // ... (backward: fewer than 4 x 148 SMs, below which the selector has to take
                                                  //     one large CTA per SM; cut until there are that many rows --
                                                  //     (256, 2^20) backward fp32 6336 -> 6633, bf16 5898 -> 6234; forward loses) ...
constexpr int64_t kSuperChunkMinRow = 1 << 17;    // ... each at least this long
constexpr int64_t kSuperChunkMinLen = 1 << 15;    // a super-chunk is at least this long
constexpr int64_t kSuperChunkTargetRows = 1024;   // cut until there are about this many independent rows
constexpr size_t kSuperChunkRecordBytes = 2 * kSuperChunkTargetRows * 16 + 256;

int pick_super_chunks(int kind, bool bwd, int dtype, int64_t numseq, int64_t seqlen, int64_t row_stride, const void* const* ptrs,
                      int nptrs, const Options& opt, bool plain)
{
    if (opt.super_chunks == 0 || opt.super_chunks == 1) return 1;
    if (!plain || kind != LINREC_KIND_PIPE || opt.logc || dtype == LINREC_DTYPE_F64) return 1;
    if (opt.memcode >= 0 && opt.memcode != 1) return 1;
    if (numseq <= 0 || seqlen <= 0 || (row_stride != seqlen && numseq != 1)) return 1;
    int64_t V = 1;
    if (opt.super_chunks > 1) {
        V = opt.super_chunks;
        if (V & (V - 1)) return 1;                 // powers of two only
        if (numseq * V > 2 * kSuperChunkTargetRows) return 1;
    } else {
        if (seqlen < kSuperChunkMinRow) return 1;
        if (numseq < kSuperChunkMaxRows) {
            while (numseq * V < kSuperChunkTargetRows) V <<= 1;
        } else if (bwd && numseq < kSuperChunkMaxRowsBwd) {
            while (numseq * V < kSuperChunkMaxRowsBwd) V <<= 1;
        } else {
            return 1;
        }
    }
    const int64_t line = 128 / (dtype == LINREC_DTYPE_F32 ? 4 : 2);
    while (V > 1 && (seqlen % V != 0 || seqlen / V < kSuperChunkMinLen || (seqlen / V) % line != 0)) V >>= 1;
    if (V < 2) return 1;
    if (!tma_eligible(dtype, numseq * V, seqlen / V, seqlen / V, ptrs, nptrs)) return 1;
    return (int)V;
}

int launch_scan(int kind, bool bwd, const void* in0, const void* c, const void* yin, void* out0, void* out1,
                float* carry_out, int carry_stride, int open_start, const void* exchange, uint32_t px_epoch, int64_t numseq,
                int64_t seqlen, int64_t row_stride, int reverse, int dtype, const linrec_opts* opts, void* workspace,
                size_t workspace_bytes, void* stream)
{
    Options opt;
    if (parse_options(opts, opt) == LINREC_OK && numseq > 0 && seqlen > 0 && in0 && c && out0 && workspace) {
        const void* ptrs[5] = {in0, c, out0, bwd ? yin : in0, bwd ? out1 : out0};
        const bool plain = !carry_out && !exchange && !open_start;
        const int V = (!bwd || (yin && out1)) ? pick_super_chunks(kind, bwd, dtype, numseq, seqlen, row_stride, ptrs, 5, opt, plain) : 1;
        const size_t rec_bytes = (size_t)round_up(numseq * V * 16, 256);
        if (V > 1 && workspace_bytes > rec_bytes + linrec::kHeaderBytes) {
            const size_t main_bytes = (workspace_bytes - rec_bytes) & ~(size_t)255;
            float* records = reinterpret_cast<float*>(static_cast<char*>(workspace) + main_bytes);
            const int64_t ns = numseq * V, len = seqlen / V;
            const int rc = launch_scan_direct(kind, bwd, in0, c, yin, out0, out1, records, bwd ? 4 : 2, 0, nullptr, 0u, ns, len,
                                              len, reverse, dtype, opts, workspace, main_bytes, stream, V);
            if (rc == LINREC_OK)
                return launch_fixup(bwd, in0, out0, out1, c, yin, records, nullptr, 0u, nullptr, 0, ns, len, len, reverse, dtype,
                                    0, V, stream, V, opt.fixup_threads);
            if (rc != LINREC_ERR_WORKSPACE) return rc;
            // the workspace holds the plain scan but not the records as well: scan the rows as they are
        }
    }
    return launch_scan_direct(kind, bwd, in0, c, yin, out0, out1, carry_out, carry_stride, open_start, exchange, px_epoch,
                              numseq, seqlen, row_stride, reverse, dtype, opts, workspace, workspace_bytes, stream);
}
}  // namespace

// ---- scan along the middle axis of (nb, seqlen, nchan) -------------------------------------------------
namespace {
const std::vector<ColVariant>& col_variants()
{
    static const std::vector<ColVariant> v = [] {
        std::vector<ColVariant> t;
        add_col_variants_0(t);
        add_col_variants_1(t);
        return t;
    }();
    return v;
}

struct ColPlan {
    const ColVariant* v = nullptr;
    int DC = 0, dtiles = 0, nq = 0, k = 0, gens = 0;
    long long units = 0, njobs = 0;
};

// Default tile shapes, widest first, with the CTAs per SM their shared memory allows.  The job
// count is sized for 148 SMs, fixed, so that the workspace a problem needs does not depend on the
// device the size query runs on.
struct ColShape {
    int NT, LC, S_fwd, S_bwd, ctas_per_sm;
};
constexpr ColShape kColShapes[3] = {{128, 32, 3, 2, 2}, {64, 64, 3, 2, 2}, {32, 64, 3, 2, 4}};
constexpr long long kColSMs = 148;

int make_col_plan(ColPlan& pl, bool bwd, int dtype, int64_t nb, int64_t seqlen, int64_t nchan, const Options& opt,
                  int max_smem)
{
    const int di = dtype == LINREC_DTYPE_F32 ? 0 : (dtype == LINREC_DTYPE_BF16 ? 1 : 2);
    const int per_word = di == 0 ? 1 : 2;
    int NT = opt.NT, LC = opt.LC, S = opt.S;
    // 0 = undecided, 1 = chained jobs of several chunks, 2 = one job per column, 3 = every chunk a job
    int mode = 0;
    long long slots = 2 * kColSMs;
    if (NT < 0 && LC < 0 && S < 0) {
        // A job waits for the inclusive value of its predecessor in the same column, which was handed
        // out `units` tickets earlier; that wait is free only if there are clearly more columns than
        // resident CTAs.  So: the widest tile that still leaves 1.25 columns per resident CTA.
        const ColShape* pick = nullptr;
        for (const ColShape& c : kColShapes) {
            const long long dc = (long long)c.NT * per_word;
            const long long u = nb * ceil_div(nchan, dc);
            // a tile much wider than the channel axis would scan mostly padding
            if (4 * ceil_div(nchan, dc) * dc > 5 * nchan && &c != &kColShapes[2]) continue;
            if (4 * u >= 5 * kColSMs * c.ctas_per_sm) {
                pick = &c;
                mode = 1;
                break;
            }
        }
        if (!pick) {
            // Fewer columns than that: the narrowest tile, and every column gets a CTA of its own for
            // its whole length, so that nobody waits for anybody (measured 2 to 4 times faster than
            // cutting such columns into chunks linked by look-back, whose dependent descriptor loads
            // then dominate).  Only with a handful of columns does the sequence axis have to supply
            // the parallelism (decoupled look-back); callers that can afford transposed copies are
            // better off with the last-axis kernels there.
            pick = &kColShapes[2];
            const long long u = nb * ceil_div(nchan, (int64_t)pick->NT * per_word);
            mode = u >= 64 ? 2 : 3;
        }
        NT = pick->NT; LC = pick->LC; S = bwd ? pick->S_bwd : pick->S_fwd;
        slots = kColSMs * pick->ctas_per_sm;
    }
    for (const ColVariant& v : col_variants()) {
        if (!((NT < 0 || v.NT == NT) && (LC < 0 || v.LC == LC) && (S < 0 || v.S == S))) continue;
        if (!v.fn[di][bwd][0] || v.smem[di][bwd] > (size_t)max_smem) continue;
        pl.v = &v;
        break;
    }
    if (!pl.v) return LINREC_ERR_NOT_IMPLEMENTED;
    pl.DC = pl.v->NT * per_word;
    pl.dtiles = (int)ceil_div(nchan, pl.DC);
    pl.units = nb * pl.dtiles;
    pl.nq = (int)ceil_div(seqlen, pl.v->LC);
    int k = opt.K;
    if (k < 0) {
        if (mode == 0) mode = 4 * pl.units >= 5 * slots ? 1 : (pl.units >= 64 ? 2 : 3);
        if (mode == 1) {
            // about 32 jobs per resident CTA, so that the last round is short, but at least 4 chunks
            // per job, so that the hand-over between jobs stays a small part of a job
            long long gens = (32 * slots + pl.units - 1) / pl.units;
            if (gens > pl.nq / 4) gens = pl.nq / 4;
            if (gens < 1) gens = 1;
            k = (int)ceil_div(pl.nq, gens);
        } else {
            k = mode == 2 ? pl.nq : 1;
        }
    }
    if (k == 0 || k > pl.nq) k = pl.nq;
    pl.k = k;
    pl.gens = (int)ceil_div(pl.nq, k);
    pl.njobs = pl.units * pl.gens;
    if (pl.njobs >= 0x7ff00000LL) return LINREC_ERR_INVALID_ARG;   // tickets are 32-bit
    return LINREC_OK;
}

size_t col_workspace_need(const ColPlan& pl)
{
    size_t n = linrec::kHeaderBytes;
    if (pl.gens > 1) n += (size_t)pl.njobs * (size_t)pl.DC * sizeof(TileDesc);
    return n;
}

bool col_eligible(int dtype, int64_t nb, int64_t seqlen, int64_t nchan, const void* const* ptrs, int nptrs)
{
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    if ((nchan * sz) % 16 != 0) return false;
    if (nb > 0x7fffffffLL || seqlen > 0x7fffffffLL - 1024 || nchan > 0x7fffffffLL) return false;
    if ((uint64_t)nchan * sz >= (1ull << 40) || (uint64_t)nchan * (uint64_t)seqlen * sz >= (1ull << 40)) return false;
    for (int i = 0; i < nptrs; ++i)
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 != 0) return false;
    return true;
}

// Rank-3 view (channels, positions, batch) of a contiguous (nb, seqlen, nchan) tensor, no swizzle;
// box = (DC channels, LC positions, 1).  Out-of-range elements read as zero and are not written.
int make_col_map(CUtensorMap* map, const void* ptr, int dtype, int64_t nb, int64_t seqlen, int64_t nchan, int box_chan,
                 int box_rows, int l2_promotion)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        note_cuda_error("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled not found");
        return LINREC_ERR_CUDA;
    }
    const int sz = dtype == LINREC_DTYPE_F32 ? 4 : 2;
    const cuuint64_t dims[3] = {(cuuint64_t)nchan, (cuuint64_t)seqlen, (cuuint64_t)nb};
    const cuuint64_t strides[2] = {(cuuint64_t)nchan * sz, (cuuint64_t)nchan * (cuuint64_t)seqlen * sz};
    const cuuint32_t box[3] = {(cuuint32_t)box_chan, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, dtype == LINREC_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == LINREC_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE,
                           l2_promotion == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                           : l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                           : l2_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof(msg), "driver error %d", (int)r);
        note_cuda_error("cuTensorMapEncodeTiled", msg);
        return LINREC_ERR_CUDA;
    }
    return LINREC_OK;
}

int launch_col(bool bwd, const void* in0, const void* c, const void* yin, void* out0, void* out1, int64_t nb,
               int64_t seqlen, int64_t nchan, int reverse, int dtype, const linrec_opts* opts, void* workspace,
               size_t workspace_bytes, void* stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype != LINREC_DTYPE_F32 && dtype != LINREC_DTYPE_BF16 && dtype != LINREC_DTYPE_F16) return LINREC_ERR_NOT_IMPLEMENTED;
    if (nb < 0 || seqlen < 0 || nchan < 0) return LINREC_ERR_INVALID_ARG;
    Options opt;
    int rc = parse_options(opts, opt);
    if (rc != LINREC_OK) return rc;
    if (nb == 0 || seqlen == 0 || nchan == 0) return LINREC_OK;
    const void* ptrs[5] = {in0, c, out0, bwd ? yin : in0, bwd ? out1 : out0};
    for (int i = 0; i < 5; ++i)
        if (!ptrs[i]) return LINREC_ERR_INVALID_ARG;
    if (!col_eligible(dtype, nb, seqlen, nchan, ptrs, 5)) return LINREC_ERR_UNALIGNED;
    DeviceInfo dev;
    rc = device_info(dev);
    if (rc != LINREC_OK) return rc;
    ColPlan pl;
    rc = make_col_plan(pl, bwd, dtype, nb, seqlen, nchan, opt, dev.max_smem_optin);
    if (rc != LINREC_OK) return rc;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0 || workspace_bytes < col_workspace_need(pl))
        return LINREC_ERR_WORKSPACE;

    const int di = dtype == LINREC_DTYPE_F32 ? 0 : (dtype == LINREC_DTYPE_BF16 ? 1 : 2);
    const bool asc = bwd ? (reverse != 0) : (reverse == 0);
    linrec::ColParams p{};
    p.nb = nb; p.seqlen = seqlen; p.nchan = nchan;
    p.dtiles = pl.dtiles; p.units = pl.units; p.nq = pl.nq; p.k_chunks = pl.k; p.gens = pl.gens; p.njobs = pl.njobs;
    p.header = static_cast<uint32_t*>(workspace);
    p.desc = reinterpret_cast<TileDesc*>(static_cast<char*>(workspace) + linrec::kHeaderBytes);
    p.wait_budget = (long long)opt.wait_budget_ms * (long long)dev.clock_khz;
    p.first_ticket = (uint32_t)opt.first_ticket;
    p.logc = opt.logc;
    p.c_raw = c;

    const ColFn fn = pl.v->fn[di][bwd][asc];
    const size_t smem = pl.v->smem[di][bwd];
    int occ = 0;
    rc = occupancy(reinterpret_cast<const void*>(fn), pl.v->NT + 32, smem, occ);
    if (rc != LINREC_OK) return rc;
    if (opt.ctas_per_sm > 0 && opt.ctas_per_sm < occ) occ = opt.ctas_per_sm;
    long long grid = (long long)dev.sm_count * occ;
    if (grid > pl.njobs) grid = pl.njobs;

    CUtensorMap m[5];
    const void* src[5] = {in0, c, bwd ? yin : c, out0, bwd ? out1 : out0};
    for (int i = 0; i < 5; ++i) {
        rc = make_col_map(&m[i], src[i], dtype, nb, seqlen, nchan, pl.DC, pl.v->LC, opt.l2_promotion);
        if (rc != LINREC_OK) return rc;
    }
    fn<<<(unsigned)grid, pl.v->NT + 32, smem, stream>>>(m[0], m[1], m[2], m[3], m[4], p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return launch_result("kernel launch");
}
}  // namespace

// ---- built-in scratch buffer ------------------------------------------------------------------------
// The buffer lives in the library's device image, so no call ever has to allocate.  In host code
// the name below is only a handle for the runtime: the device address has to be asked for with
// cudaGetSymbolAddress, once per device and with that device current, and it is that address --
// never the host-side symbol -- that goes to the kernels.
static __device__ __align__(256) unsigned char g_static_scratch[LINREC_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

int static_scratch_address(void** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return LINREC_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return LINREC_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return LINREC_ERR_CUDA;
        }
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return LINREC_OK;
}
}  // namespace


// =================================================================================================
//  C ABI
// =================================================================================================
extern "C" {

size_t linrec_b200_workspace_size(int64_t numseq, int64_t seqlen, int dtype)
{
    (void)dtype;
    size_t n = linrec::kHeaderBytes;
    if (numseq > 0 && seqlen > 0) {
        // the smallest tile any variant uses bounds the number of chained tiles from above
        int tmin = 1 << 30;
        for (const TmaVariant& v : tma_variants()) tmin = v.E * v.NT < tmin ? v.E * v.NT : tmin;
        for (const GenericVariant& v : generic_variants()) tmin = v.E * v.NT < tmin ? v.E * v.NT : tmin;
        for (const GenericVariant& v : async_variants()) tmin = v.E * v.NT < tmin ? v.E * v.NT : tmin;
        for (const GenericVariant& v : word_variants()) tmin = v.E * v.NT < tmin ? v.E * v.NT : tmin;
        if (seqlen > tmin) n += (size_t)numseq * (size_t)ceil_div(seqlen, tmin) * sizeof(TileDesc);
        // few very long rows may be cut into super-chunks: their records and a few more descriptors
        if (numseq < kSuperChunkMaxRowsBwd && seqlen >= kSuperChunkMinRow) n += 2 * kSuperChunkRecordBytes;
    }
    return (size_t)round_up((int64_t)n, 256);
}

int linrec_b200_fwd(int kind, const void* x, const void* c, void* y, int64_t numseq, int64_t seqlen,
                    int64_t row_stride, int reverse, int dtype, const linrec_opts* opts, void* workspace,
                    size_t workspace_bytes, void* stream)
{
    return launch_scan(kind, false, x, c, nullptr, y, nullptr, nullptr, 0, 0, nullptr, 0u, numseq, seqlen, row_stride, reverse,
                       dtype, opts, workspace, workspace_bytes, stream);
}

int linrec_b200_bwd(int kind, const void* dy, const void* c, const void* y, void* dx, void* dc, int64_t numseq,
                    int64_t seqlen, int64_t row_stride, int reverse, int dtype, const linrec_opts* opts,
                    void* workspace, size_t workspace_bytes, void* stream)
{
    return launch_scan(kind, true, dy, c, y, dx, dc, nullptr, 0, 0, nullptr, 0u, numseq, seqlen, row_stride, reverse, dtype, opts,
                       workspace, workspace_bytes, stream);
}

int linrec_b200_status(const void* workspace, void* stream)
{
    if (!workspace) {
        // the built-in buffer of the current device (linrec_b200_fwd_static)
        void* scratch = nullptr;
        const int rc = static_scratch_address(&scratch);
        if (rc != LINREC_OK) return rc;
        workspace = scratch;
    }
    uint32_t words[2] = {0, 0};
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return LINREC_ERR_CUDA;
    if (cudaMemcpy(words, workspace, sizeof(words), cudaMemcpyDeviceToHost) != cudaSuccess) return LINREC_ERR_CUDA;
    if (words[1] == 0) return LINREC_OK;
    // the word is sticky until it has been read: clear it now
    if (cudaMemset(static_cast<char*>(const_cast<void*>(workspace)) + sizeof(uint32_t), 0, sizeof(uint32_t)) != cudaSuccess)
        return LINREC_ERR_CUDA;
    return LINREC_ERR_TIMEOUT;
}

int linrec_b200_attrs(int kind, int fwd, int dtype, const linrec_opts* opts, const char** names, int* values, int cap)
{
    if (!names || !values || cap <= 0) return LINREC_ERR_INVALID_ARG;
    if (dtype != LINREC_DTYPE_F32 && dtype != LINREC_DTYPE_BF16 && dtype != LINREC_DTYPE_F16) return LINREC_ERR_NOT_IMPLEMENTED;
    Options opt;
    int rc = parse_options(opts, opt);
    if (rc != LINREC_OK) return rc;
    const int di = dtype == LINREC_DTYPE_F32 ? 0 : (dtype == LINREC_DTYPE_BF16 ? 1 : 2);
    const bool bwd = !fwd;
    const void* fn = nullptr;
    int E = 0, NT = 0, S = 0, OB = 0, memcode = 0;
    size_t dyn = 0;
    if (kind == LINREC_KIND_REF) {
        fn = di == 0 ? (bwd ? (const void*)linrec::linrec_seq_kernel<float, true> : (const void*)linrec::linrec_seq_kernel<float, false>)
                     : di == 1 ? (bwd ? (const void*)linrec::linrec_seq_kernel<__nv_bfloat16, true> : (const void*)linrec::linrec_seq_kernel<__nv_bfloat16, false>)
                               : (bwd ? (const void*)linrec::linrec_seq_kernel<__half, true> : (const void*)linrec::linrec_seq_kernel<__half, false>);
        E = 1; NT = 128;
    } else {
        // attributes are reported for an aligned problem unless memcode=0 is asked for
        Plan pl;
        Options o2 = opt;
        if (o2.memcode < 0) o2.memcode = 1;
        static const double dummy_align[2] = {0, 0};
        const void* ptrs[1] = {reinterpret_cast<const void*>((reinterpret_cast<uintptr_t>(dummy_align) + 15) & ~(uintptr_t)15)};
        DeviceInfo dev;
        rc = device_info(dev);
        if (rc != LINREC_OK) return rc;
        rc = make_plan(pl, LINREC_KIND_PIPE, bwd, dtype, 1024, 1 << 20, 1 << 20, ptrs, 0, o2, dev.max_smem_optin, dev.sm_count);
        if (rc != LINREC_OK) return rc;
        if (pl.tma) {
            fn = reinterpret_cast<const void*>(pl.tv->fn[di][bwd][1]);
            E = pl.tv->E; NT = pl.tv->NT; S = pl.tv->S; OB = pl.tv->OB; memcode = 1;
            dyn = pl.tv->smem[di][bwd];
        } else {
            fn = reinterpret_cast<const void*>(pl.gv->fn[di][bwd][1]);
            E = pl.gv->E; NT = pl.gv->NT; S = pl.gv->S; OB = 0; memcode = pl.memcode;
            dyn = pl.gv->smem[di][bwd];
        }
    }
    cudaFuncAttributes a;
    if (cudaFuncGetAttributes(&a, fn) != cudaSuccess) {
        cudaGetLastError();
        return LINREC_ERR_CUDA;
    }
    int occ = 0;
    if (occupancy(fn, NT, dyn, occ) != LINREC_OK) occ = 0;
    const char* nm[] = {"sharedSizeBytes", "constSizeBytes", "localSizeBytes", "maxThreadsPerBlock", "numRegs",
                        "ptxVersion", "binaryVersion", "maxDynamicSharedSizeBytes", "dynamicSharedSizeBytes",
                        "residentBlocksPerSM", "kElemsPerThread", "kThreadsPerBlock", "kStages", "kOutBuffers", "memcode"};
    const int vl[] = {(int)a.sharedSizeBytes, (int)a.constSizeBytes, (int)a.localSizeBytes, a.maxThreadsPerBlock, a.numRegs,
                      a.ptxVersion, a.binaryVersion, a.maxDynamicSharedSizeBytes, (int)dyn, occ, E, NT, S, OB, memcode};
    const int n = (int)(sizeof(vl) / sizeof(vl[0]));
    int w = 0;
    for (; w < n && w < cap; ++w) {
        names[w] = nm[w];
        values[w] = vl[w];
    }
    return w;
}

int linrec_b200_config_names(const char** names, int cap)
{
    if (names)
        for (int i = 0; i < kNumConfigNames && i < cap; ++i) names[i] = kConfigNames[i];
    return kNumConfigNames;
}

int linrec_b200_config_list(int* values, int cap_rows)
{
    int row = 0;
    auto put = [&](int E, int NT, int S, int OB, int memcode) {
        if (values && row < cap_rows) {
            int* r = values + (size_t)row * kNumConfigNames;
            r[0] = E; r[1] = NT; r[2] = S; r[3] = OB; r[4] = memcode;
        }
        ++row;
    };
    for (const TmaVariant& v : tma_variants()) put(v.E, v.NT, v.S, v.OB, 1);
    for (const GenericVariant& v : generic_variants()) put(v.E, v.NT, 1, 0, 0);
    for (const GenericVariant& v : async_variants()) put(v.E, v.NT, v.S, 0, 2);
    for (const GenericVariant& v : word_variants()) put(v.E, v.NT, v.S, 0, 3);
    return row;
}

int linrec_b200_fwd_carry(const void* x, const void* c, void* y, float* records, int64_t numseq, int64_t seqlen,
                          int64_t row_stride, int reverse, int dtype, int shard, int nshards, const linrec_opts* opts,
                          void* workspace, size_t workspace_bytes, void* stream)
{
    if (!records && numseq > 0 && seqlen > 0) return LINREC_ERR_INVALID_ARG;
    if (nshards < 1 || shard < 0 || shard >= nshards) return LINREC_ERR_INVALID_ARG;
    const int open = holds_scan_start(reverse == 0, shard, nshards) ? 0 : 1;
    return launch_scan(LINREC_KIND_PIPE, false, x, c, nullptr, y, nullptr, records, 2, open, nullptr, 0u, numseq, seqlen, row_stride,
                       reverse, dtype, opts, workspace, workspace_bytes, stream);
}

int linrec_b200_fwd_fixup(const void* x, void* y, const void* c, const float* records, int64_t numseq, int64_t seqlen,
                          int64_t row_stride, int reverse, int dtype, int shard, int nshards, void* stream)
{
    return launch_fixup(false, x, y, nullptr, c, nullptr, records, nullptr, 0u, nullptr, 0, numseq, seqlen, row_stride, reverse, dtype,
                        shard, nshards, stream);
}

int linrec_b200_bwd_carry(const void* dy, const void* c, const void* y, void* dx, void* dc, float* records,
                          int64_t numseq, int64_t seqlen, int64_t row_stride, int reverse, int dtype, int shard,
                          int nshards, const linrec_opts* opts, void* workspace, size_t workspace_bytes, void* stream_)
{
    if (!records && numseq > 0 && seqlen > 0) return LINREC_ERR_INVALID_ARG;
    if (nshards < 1 || shard < 0 || shard >= nshards) return LINREC_ERR_INVALID_ARG;
    const bool asc = reverse != 0;   // the gradient scan runs against the forward direction
    const int open = holds_scan_start(asc, shard, nshards) ? 0 : 1;
    // the scan kernel writes the whole record, edge elements included
    return launch_scan(LINREC_KIND_PIPE, true, dy, c, y, dx, dc, records, 4, open, nullptr, 0u, numseq, seqlen, row_stride,
                       reverse, dtype, opts, workspace, workspace_bytes, stream_);
}

int linrec_b200_bwd_fixup(const void* dy, void* dx, void* dc, const void* c, const void* y, const float* records,
                          int64_t numseq, int64_t seqlen, int64_t row_stride, int reverse, int dtype, int shard, int nshards,
                          void* stream)
{
    return launch_fixup(true, dy, dx, dc, c, y, records, nullptr, 0u, nullptr, 0, numseq, seqlen, row_stride, reverse, dtype, shard, nshards,
                        stream);
}

// ---- sequence sharding with a peer exchange instead of a collective call ---------------------------------
size_t linrec_b200_exchange_size(int64_t max_rows, int nranks)
{
    if (max_rows < 1 || nranks < 1 || nranks > linrec::kMaxPeers) return 0;
    return linrec::px_total_bytes(max_rows, nranks);
}

int linrec_b200_exchange_init(void* local_buf, void* const* peer_bufs, int rank, int nranks, int64_t max_rows, void* stream_)
{
    if (!local_buf || !peer_bufs || nranks < 1 || nranks > linrec::kMaxPeers || rank < 0 || rank >= nranks || max_rows < 1)
        return LINREC_ERR_INVALID_ARG;
    linrec::PeerTableArg a{};
    for (int i = 0; i < nranks; ++i) {
        if (!peer_bufs[i] || reinterpret_cast<uintptr_t>(peer_bufs[i]) % 256 != 0) return LINREC_ERR_INVALID_ARG;
        a.t.base[i] = peer_bufs[i];
    }
    if (peer_bufs[rank] != local_buf) return LINREC_ERR_INVALID_ARG;
    a.t.nranks = nranks; a.t.me = rank; a.t.max_rows = max_rows;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaMemsetAsync(local_buf, 0, linrec::px_total_bytes(max_rows, nranks), stream) != cudaSuccess) {
        cudaGetLastError();
        return LINREC_ERR_CUDA;
    }
    linrec::linrec_exchange_init_kernel<<<1, 32, 0, stream>>>(static_cast<linrec::PeerTable*>(local_buf), a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return launch_result("kernel launch");
}

int linrec_b200_fwd_seq_p2p(const void* x, const void* c, void* y, int64_t numseq, int64_t seqlen, int64_t row_stride,
                            int reverse, int dtype, int shard, int nshards, void* exchange, uint32_t epoch,
                            const linrec_opts* opts, void* workspace, size_t workspace_bytes, void* stream)
{
    if (!exchange || epoch == 0 || nshards < 1 || nshards > linrec::kMaxPeers || shard < 0 || shard >= nshards)
        return LINREC_ERR_INVALID_ARG;
    Options opt;
    int rc = parse_options(opts, opt);
    if (rc != LINREC_OK) return rc;
    const int open = holds_scan_start(reverse == 0, shard, nshards) ? 0 : 1;
    if (opt.p2p_phase != 2)
        rc = launch_scan(LINREC_KIND_PIPE, false, x, c, nullptr, y, nullptr, nullptr, 0, open, exchange, epoch, numseq, seqlen,
                         row_stride, reverse, dtype, opts, workspace, workspace_bytes, stream);
    if (rc != LINREC_OK || numseq == 0 || seqlen == 0 || opt.p2p_phase == 1) return rc;
    return launch_fixup(false, x, y, nullptr, c, nullptr, nullptr, exchange, epoch, static_cast<uint32_t*>(workspace) + 1,
                        opt.peer_wait_budget_ms, numseq, seqlen, row_stride, reverse, dtype, shard, nshards, stream);
}

int linrec_b200_bwd_seq_p2p(const void* dy, const void* c, const void* y, void* dx, void* dc, int64_t numseq,
                            int64_t seqlen, int64_t row_stride, int reverse, int dtype, int shard, int nshards,
                            void* exchange, uint32_t epoch, const linrec_opts* opts, void* workspace, size_t workspace_bytes,
                            void* stream)
{
    if (!exchange || epoch == 0 || nshards < 1 || nshards > linrec::kMaxPeers || shard < 0 || shard >= nshards)
        return LINREC_ERR_INVALID_ARG;
    Options opt;
    int rc = parse_options(opts, opt);
    if (rc != LINREC_OK) return rc;
    const bool asc = reverse != 0;
    const int open = holds_scan_start(asc, shard, nshards) ? 0 : 1;
    if (opt.p2p_phase != 2)
        rc = launch_scan(LINREC_KIND_PIPE, true, dy, c, y, dx, dc, nullptr, 0, open, exchange, epoch, numseq, seqlen, row_stride,
                         reverse, dtype, opts, workspace, workspace_bytes, stream);
    if (rc != LINREC_OK || numseq == 0 || seqlen == 0 || opt.p2p_phase == 1) return rc;
    return launch_fixup(true, dy, dx, dc, c, y, nullptr, exchange, epoch, static_cast<uint32_t*>(workspace) + 1,
                        opt.peer_wait_budget_ms, numseq, seqlen, row_stride, reverse, dtype, shard, nshards, stream);
}

int linrec_b200_fwd_static(const void* x, const void* c, void* y, int64_t numseq, int64_t seqlen,
                           int64_t row_stride, int reverse, int dtype, void* stream)
{
    const void* ptrs[3] = {x, c, y};
    if (dtype == LINREC_DTYPE_F64) return LINREC_ERR_NOT_IMPLEMENTED;
    int rc = check_common(ptrs, 3, numseq, seqlen, row_stride, dtype);
    if (rc != LINREC_OK) return rc;
    if (numseq == 0 || seqlen == 0) return LINREC_OK;
    // how much scratch this very problem needs, with the same plan the launch below will make
    DeviceInfo dev;
    rc = device_info(dev);
    if (rc != LINREC_OK) return rc;
    Plan pl;
    const void* all[5] = {x, c, y, x, y};
    rc = make_plan(pl, LINREC_KIND_PIPE, false, dtype, numseq, seqlen, row_stride, all, 5, Options{}, dev.max_smem_optin, dev.sm_count);
    if (rc != LINREC_OK) return rc;
    if (workspace_need(pl) > (size_t)LINREC_STATIC_SCRATCH_BYTES) return LINREC_ERR_SCRATCH_LIMIT;
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != LINREC_OK) return rc;
    // Everybody shares this buffer and nobody can re-zero it from outside, so what a launch needs at
    // zero is cleared here, on the caller's stream, ahead of the kernel: header word 0 (ticket counter)
    // and word 3 (CTAs finished).  Word 1 (the sticky status) and word 2 (the epoch) must survive:
    // resetting the epoch would make the descriptors of earlier launches valid again.  Two 4-byte
    // memsets, no allocation.
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, sizeof(uint32_t), st) != cudaSuccess ||
        cudaMemsetAsync(static_cast<uint32_t*>(scratch) + 3, 0, sizeof(uint32_t), st) != cudaSuccess) {
        note_cuda_error("cudaMemsetAsync", cudaGetErrorString(cudaGetLastError()));
        return LINREC_ERR_CUDA;
    }
    return launch_scan(LINREC_KIND_PIPE, false, x, c, nullptr, y, nullptr, nullptr, 0, 0, nullptr, 0u, numseq, seqlen, row_stride,
                       reverse, dtype, nullptr, scratch, (size_t)LINREC_STATIC_SCRATCH_BYTES, stream);
}

int linrec_b200_static_workspace(void** workspace, size_t* bytes)
{
    if (!workspace || !bytes) return LINREC_ERR_INVALID_ARG;
    void* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != LINREC_OK) return rc;
    *workspace = scratch;
    *bytes = (size_t)LINREC_STATIC_SCRATCH_BYTES;
    return LINREC_OK;
}

uint64_t linrec_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

/* ---- scan along the middle axis of a contiguous (nb, seqlen, nchan) tensor ------------------------------ */
size_t linrec_b200_dim_workspace_size(int bwd, int64_t nb, int64_t seqlen, int64_t nchan, int dtype,
                                      const linrec_opts* opts)
{
    Options opt;
    if (parse_options(opts, opt) != LINREC_OK) return 0;
    if (nb <= 0 || seqlen <= 0 || nchan <= 0) return (size_t)linrec::kHeaderBytes;
    ColPlan pl;
    if (make_col_plan(pl, bwd != 0, dtype, nb, seqlen, nchan, opt, 232448) != LINREC_OK) return 0;
    return (size_t)round_up((int64_t)col_workspace_need(pl), 256);
}

int linrec_b200_fwd_dim(const void* x, const void* c, void* y, int64_t nb, int64_t seqlen, int64_t nchan, int reverse,
                        int dtype, const linrec_opts* opts, void* workspace, size_t workspace_bytes, void* stream)
{
    return launch_col(false, x, c, nullptr, y, nullptr, nb, seqlen, nchan, reverse, dtype, opts, workspace,
                      workspace_bytes, stream);
}

int linrec_b200_bwd_dim(const void* dy, const void* c, const void* y, void* dx, void* dc, int64_t nb, int64_t seqlen,
                        int64_t nchan, int reverse, int dtype, const linrec_opts* opts, void* workspace,
                        size_t workspace_bytes, void* stream)
{
    return launch_col(true, dy, c, y, dx, dc, nb, seqlen, nchan, reverse, dtype, opts, workspace, workspace_bytes,
                      stream);
}

const char* linrec_b200_last_cuda_error(void) { return g_last_cuda_error; }

const char* linrec_b200_strerror(int code)
{
    switch (code) {
        case LINREC_OK: return "ok";
        case LINREC_ERR_INVALID_ARG: return "invalid argument";
        case LINREC_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case LINREC_ERR_NOT_IMPLEMENTED: return "no compiled variant for these options";
        case LINREC_ERR_CUDA: return "a CUDA call failed";
        case LINREC_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case LINREC_ERR_TOO_LONG: return "row does not fit one tile";
        case LINREC_ERR_UNALIGNED: return "this copy path needs 16-byte aligned rows (bulk copies along the last axis: whole 128-byte lines)";
        case LINREC_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the 1 MiB built into the library (use linrec_b200_fwd with a workspace)";
        default: return "unknown status";
    }
}

int linrec_b200_version(void) { return 200; }

}  // extern "C"
