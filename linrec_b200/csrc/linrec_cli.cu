// Standalone verify/bench harness for the C ABI (no Python, no torch): the target for profilers
// and the tuning sweep.  Counterpart of the reference's linrec/impl/cuda/executable.cpp:16-68,
// which runs its ref and pipe operators on random data and prints registers and max error.
//
//   linrec_cli --numseq 512 --seqlen 65536 [--reverse] [--bwd] [--dtype f32|bf16|f16]
//              [--clo 0 --chi 1] [--stride N] [--iters 20 --warmup 3] [--flush]
//              [--opt name=value ...] [--sweep] [--no-verify] [--kind pipe|tile|ref] [--dump PREFIX]
//
// --dump writes the operands and the results of the last measured configuration as raw arrays, so that
// a checker outside this program (the CPU oracle of the test-suite) can judge them.
//
// Prints one JSON object per measured configuration.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "linrec_b200.h"

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) {                                                              \
            fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(2);                                                                          \
        }                                                                                     \
    } while (0)

// ---- deterministic data ---------------------------------------------------------------------------
__device__ inline uint64_t mix64(uint64_t z)
{
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

template <typename T>
__device__ inline T cast_to(float v);
template <>
__device__ inline float cast_to<float>(float v) { return v; }
template <>
__device__ inline __nv_bfloat16 cast_to<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <>
__device__ inline __half cast_to<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__device__ inline float cast_from(T v);
template <>
__device__ inline float cast_from<__half>(__half v) { return __half2float(v); }
template <>
__device__ inline float cast_from<float>(float v) { return v; }
template <>
__device__ inline float cast_from<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// normal(0,1) when lo > hi is passed as (1, 0); else uniform [lo, hi)
template <typename T>
__global__ void fill_kernel(T* p, size_t n, uint64_t seed, float lo, float hi, int normal)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t r = mix64(seed * 0x100000001b3ull + i);
        const float u1 = ((r >> 40) + 0.5f) * (1.0f / 16777216.0f);
        const float u2 = (((r >> 16) & 0xffffff) + 0.5f) * (1.0f / 16777216.0f);
        float v;
        if (normal) v = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        else v = lo + (hi - lo) * u1;
        p[i] = cast_to<T>(v);
    }
}

// max |a-b| and the number of elements outside |a-b| <= atol + rtol*|b|
template <typename T>
__global__ void compare_kernel(const T* a, const T* b, size_t numseq, size_t seqlen, size_t stride, float rtol,
                               float atol, float* max_abs, unsigned long long* bad)
{
    float m = 0.0f;
    unsigned long long nb = 0;
    const size_t n = numseq * seqlen;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / seqlen, col = i - r * seqlen;
        const float x = cast_from<T>(a[r * stride + col]), y = cast_from<T>(b[r * stride + col]);
        const float d = fabsf(x - y);
        if (!(d <= atol + rtol * fabsf(y))) ++nb;
        if (d > m || d != d) m = (d != d) ? INFINITY : d;
    }
    atomicMax(reinterpret_cast<int*>(max_abs), __float_as_int(m));   // valid for non-negative floats
    if (nb) atomicAdd(bad, nb);
}

__global__ void flush_kernel(float* p, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        p[i] = (float)i;
}

struct Args {
    long long numseq = 512, seqlen = 65536, stride = 0;
    long long chan = 0;   // > 0: tensor (numseq, seqlen, chan), scan along the middle axis
    int reverse = 0, bwd = 0, dtype = LINREC_DTYPE_F32, iters = 20, warmup = 3, flush = 0, sweep = 0, verify = 1;
    int kind = LINREC_KIND_PIPE;
    float clo = 0.0f, chi = 1.0f;
    std::vector<std::string> opt_names;
    std::vector<int> opt_values;
    std::string dump;     // not empty: write operands and results to <dump>.{in0,c,y,out0,out1}.bin (raw storage type)
};

static void usage()
{
    fprintf(stderr,
            "usage: linrec_cli [--numseq N] [--seqlen L] [--stride S | --chan D] [--reverse] [--bwd] [--dtype f32|bf16|f16]\n"
            "                  [--clo a --chi b] [--iters K --warmup W] [--flush] [--opt name=value ...]\n"
            "                  [--sweep] [--no-verify] [--kind pipe|tile|ref] [--dump PREFIX]\n");
}

struct Result {
    int rc = 0, status = 0;
    float ms_med = 0, ms_min = 0, max_err0 = -1, max_err1 = -1;
    unsigned long long bad0 = 0, bad1 = 0;
};

template <typename T>
static Result run_one(const Args& a, const std::vector<std::string>& names, const std::vector<int>& values,
                      T* in0, T* c, T* yfw, T* out0, T* out1, T* ref0, T* ref1, void* ws, size_t ws_bytes,
                      float* flush_buf, size_t flush_n, float* d_max, unsigned long long* d_bad)
{
    Result r;
    std::vector<const char*> np;
    for (auto& s : names) np.push_back(s.c_str());
    linrec_opts o{(int)names.size(), np.data(), values.data()};
    const linrec_opts* po = names.empty() ? nullptr : &o;
    cudaStream_t st = 0;
    auto call = [&]() -> int {
        if (a.chan > 0) {
            if (!a.bwd)
                return linrec_b200_fwd_dim(in0, c, out0, a.numseq, a.seqlen, a.chan, a.reverse, a.dtype, po, ws, ws_bytes, st);
            return linrec_b200_bwd_dim(in0, c, yfw, out0, out1, a.numseq, a.seqlen, a.chan, a.reverse, a.dtype, po, ws,
                                       ws_bytes, st);
        }
        if (!a.bwd)
            return linrec_b200_fwd(a.kind, in0, c, out0, a.numseq, a.seqlen, a.stride, a.reverse, a.dtype, po, ws, ws_bytes, st);
        return linrec_b200_bwd(a.kind, in0, c, yfw, out0, out1, a.numseq, a.seqlen, a.stride, a.reverse, a.dtype, po, ws,
                               ws_bytes, st);
    };
    const size_t total = a.chan > 0 ? (size_t)a.numseq * a.seqlen * a.chan : (size_t)a.numseq * a.stride;
    // element-wise comparison: with a channel axis the tensor is compared as rows of `chan` elements
    const long long cmp_rows = a.chan > 0 ? a.numseq * a.seqlen : a.numseq;
    const long long cmp_len = a.chan > 0 ? a.chan : a.seqlen;
    const long long cmp_stride = a.chan > 0 ? a.chan : a.stride;
    CK(cudaMemset(out0, 0xff, total * sizeof(T)));
    if (a.bwd) CK(cudaMemset(out1, 0xff, total * sizeof(T)));
    r.rc = call();
    if (r.rc != LINREC_OK) return r;
    CK(cudaDeviceSynchronize());
    r.status = linrec_b200_status(ws, st);
    if (a.verify) {
        const float rtol = a.dtype == LINREC_DTYPE_F32 ? 1e-4f : a.dtype == LINREC_DTYPE_BF16 ? 7.8125e-3f : 1.953125e-3f, atol = 1e-5f;
        float hm;
        unsigned long long hb;
        CK(cudaMemset(d_max, 0, sizeof(float)));
        CK(cudaMemset(d_bad, 0, sizeof(unsigned long long)));
        compare_kernel<T><<<1024, 256>>>(out0, ref0, cmp_rows, cmp_len, cmp_stride, rtol, atol, d_max, d_bad);
        CK(cudaMemcpy(&hm, d_max, sizeof(float), cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(&hb, d_bad, sizeof(hb), cudaMemcpyDeviceToHost));
        r.max_err0 = hm;
        r.bad0 = hb;
        if (a.bwd) {
            CK(cudaMemset(d_max, 0, sizeof(float)));
            CK(cudaMemset(d_bad, 0, sizeof(unsigned long long)));
            compare_kernel<T><<<1024, 256>>>(out1, ref1, cmp_rows, cmp_len, cmp_stride, rtol, atol, d_max, d_bad);
            CK(cudaMemcpy(&hm, d_max, sizeof(float), cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(&hb, d_bad, sizeof(hb), cudaMemcpyDeviceToHost));
            r.max_err1 = hm;
            r.bad1 = hb;
        }
    }
    for (int i = 0; i < a.warmup; ++i) call();
    std::vector<cudaEvent_t> e0(a.iters), e1(a.iters);
    for (int i = 0; i < a.iters; ++i) {
        CK(cudaEventCreate(&e0[i]));
        CK(cudaEventCreate(&e1[i]));
    }
    for (int i = 0; i < a.iters; ++i) {
        if (a.flush) flush_kernel<<<2048, 256, 0, st>>>(flush_buf, flush_n);
        CK(cudaEventRecord(e0[i], st));
        call();
        CK(cudaEventRecord(e1[i], st));
    }
    CK(cudaDeviceSynchronize());
    std::vector<float> ms(a.iters);
    for (int i = 0; i < a.iters; ++i) {
        CK(cudaEventElapsedTime(&ms[i], e0[i], e1[i]));
        cudaEventDestroy(e0[i]);
        cudaEventDestroy(e1[i]);
    }
    std::sort(ms.begin(), ms.end());
    r.ms_med = ms[ms.size() / 2];
    r.ms_min = ms[0];
    const int s2 = linrec_b200_status(ws, st);
    if (s2 != LINREC_OK) r.status = s2;
    return r;
}

// Sequential walk down the middle axis of (nb, seqlen, nchan), one thread per (batch, channel): the
// checker for the --chan mode (same arithmetic as the sequential operator of the library).
template <typename T>
__global__ void column_reference_kernel(const T* in0, const T* c, const T* yfw, T* out0, T* out1, long long nb,
                                        long long L, long long D, int reverse, int bwd)
{
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= nb * D) return;
    const long long b = i / D, d = i - b * D;
    const long long base = b * L * D + d;
    const bool asc = bwd ? (reverse != 0) : (reverse == 0);
    float v = 0.0f;
    for (long long k = 0; k < L; ++k) {
        const long long l = asc ? k : L - 1 - k;
        const long long prev = asc ? l - 1 : l + 1, next = asc ? l + 1 : l - 1;
        const long long at = base + l * D;
        if (!bwd) {
            v = k == 0 ? cast_from<T>(in0[at]) : fmaf(v, cast_from<T>(c[at]), cast_from<T>(in0[at]));
            out0[at] = cast_to<T>(v);
        } else {
            const float cp = k == 0 ? 0.0f : cast_from<T>(c[base + prev * D]);
            v = fmaf(v, cp, cast_from<T>(in0[at]));
            const float yn = (next < 0 || next >= L) ? 0.0f : cast_from<T>(yfw[base + next * D]);
            out0[at] = cast_to<T>(v);
            out1[at] = cast_to<T>(v * yn);
        }
    }
}

template <typename T>
static int run(const Args& a)
{
    const size_t total = a.chan > 0 ? (size_t)a.numseq * a.seqlen * a.chan : (size_t)a.numseq * a.stride;
    T *in0, *c, *yfw = nullptr, *out0, *out1 = nullptr, *ref0, *ref1 = nullptr;
    CK(cudaMalloc(&in0, total * sizeof(T)));
    CK(cudaMalloc(&c, total * sizeof(T)));
    CK(cudaMalloc(&out0, total * sizeof(T)));
    CK(cudaMalloc(&ref0, total * sizeof(T)));
    if (a.bwd) {
        CK(cudaMalloc(&yfw, total * sizeof(T)));
        CK(cudaMalloc(&out1, total * sizeof(T)));
        CK(cudaMalloc(&ref1, total * sizeof(T)));
    }
    size_t ws_bytes = linrec_b200_workspace_size(a.numseq, a.chan > 0 ? a.seqlen * a.chan : a.seqlen, a.dtype);
    if (a.chan > 0) {
        std::vector<const char*> np;
        for (auto& n : a.opt_names) np.push_back(n.c_str());
        linrec_opts o{(int)np.size(), np.data(), a.opt_values.data()};
        const size_t need = linrec_b200_dim_workspace_size(a.bwd, a.numseq, a.seqlen, a.chan, a.dtype, np.empty() ? nullptr : &o);
        if (need == 0) { fprintf(stderr, "no compiled variant for these options\n"); return 5; }
        if (need > ws_bytes) ws_bytes = need;
    }
    void* ws;
    CK(cudaMalloc(&ws, ws_bytes));
    CK(cudaMemset(ws, 0, ws_bytes));   // once; launches leave the workspace ready for the next one
    float* flush_buf = nullptr;
    const size_t flush_n = a.flush ? (size_t)64 << 20 : 0;   // 256 MiB of floats, twice the L2
    if (a.flush) CK(cudaMalloc(&flush_buf, flush_n * sizeof(float)));
    float* d_max;
    unsigned long long* d_bad;
    CK(cudaMalloc(&d_max, sizeof(float)));
    CK(cudaMalloc(&d_bad, sizeof(unsigned long long)));

    fill_kernel<T><<<2048, 256>>>(in0, total, 1, 0, 0, 1);
    fill_kernel<T><<<2048, 256>>>(c, total, 2, a.clo, a.chi, 0);
    CK(cudaDeviceSynchronize());
    const unsigned col_blocks = a.chan > 0 ? (unsigned)((a.numseq * a.chan + 127) / 128) : 0u;
    if (a.chan > 0) {
        if (a.bwd) {
            column_reference_kernel<T><<<col_blocks, 128>>>(in0, c, nullptr, yfw, nullptr, a.numseq, a.seqlen, a.chan, a.reverse, 0);
            fill_kernel<T><<<2048, 256>>>(in0, total, 3, 0, 0, 1);   // upstream gradient
        }
        if (a.verify) column_reference_kernel<T><<<col_blocks, 128>>>(in0, c, yfw, ref0, ref1, a.numseq, a.seqlen, a.chan, a.reverse, a.bwd);
        CK(cudaDeviceSynchronize());
    } else if (a.bwd) {
        // forward outputs feed the backward pass; made by the sequential operator
        int rc = linrec_b200_fwd(LINREC_KIND_REF, in0, c, yfw, a.numseq, a.seqlen, a.stride, a.reverse, a.dtype, nullptr, ws,
                                 ws_bytes, 0);
        if (rc) { fprintf(stderr, "reference forward failed: %s\n", linrec_b200_strerror(rc)); return 1; }
        fill_kernel<T><<<2048, 256>>>(in0, total, 3, 0, 0, 1);   // upstream gradient
    }
    if (a.verify && a.chan == 0) {
        int rc = a.bwd ? linrec_b200_bwd(LINREC_KIND_REF, in0, c, yfw, ref0, ref1, a.numseq, a.seqlen, a.stride, a.reverse,
                                         a.dtype, nullptr, ws, ws_bytes, 0)
                       : linrec_b200_fwd(LINREC_KIND_REF, in0, c, ref0, a.numseq, a.seqlen, a.stride, a.reverse, a.dtype,
                                         nullptr, ws, ws_bytes, 0);
        if (rc) { fprintf(stderr, "reference operator failed: %s\n", linrec_b200_strerror(rc)); return 1; }
        CK(cudaDeviceSynchronize());
    }

    std::vector<std::vector<int>> configs;
    std::vector<std::string> cfg_names;
    if (a.sweep) {
        const int ncol = linrec_b200_config_names(nullptr, 0);
        std::vector<const char*> nm(ncol);
        linrec_b200_config_names(nm.data(), ncol);
        for (auto s : nm) cfg_names.push_back(s);
        const int nrow = linrec_b200_config_list(nullptr, 0);
        std::vector<int> vals((size_t)nrow * ncol);
        linrec_b200_config_list(vals.data(), nrow);
        for (int r = 0; r < nrow; ++r) configs.emplace_back(vals.begin() + (size_t)r * ncol, vals.begin() + (size_t)(r + 1) * ncol);
    } else {
        configs.emplace_back();
    }

    const double elems = (double)a.numseq * (double)a.seqlen * (a.chan > 0 ? (double)a.chan : 1.0);
    const double bytes = elems * (a.bwd ? 5.0 : 3.0) * sizeof(T);
    int worst = 0;
    for (const auto& cfg : configs) {
        std::vector<std::string> names = cfg_names;
        std::vector<int> values = cfg;
        for (size_t i = 0; i < a.opt_names.size(); ++i) {
            names.push_back(a.opt_names[i]);
            values.push_back(a.opt_values[i]);
        }
        Result r = run_one<T>(a, names, values, in0, c, yfw, out0, out1, ref0, ref1, ws, ws_bytes, flush_buf, flush_n, d_max, d_bad);
        printf("{\"numseq\": %lld, \"seqlen\": %lld, \"chan\": %lld, \"stride\": %lld, \"reverse\": %d, \"bwd\": %d, \"dtype\": \"%s\", \"kind\": %d, \"opts\": {",
               a.numseq, a.seqlen, a.chan, a.stride, a.reverse, a.bwd, a.dtype == LINREC_DTYPE_F32 ? "f32" : a.dtype == LINREC_DTYPE_BF16 ? "bf16" : "f16", a.kind);
        for (size_t i = 0; i < names.size(); ++i) printf("%s\"%s\": %d", i ? ", " : "", names[i].c_str(), values[i]);
        printf("}, \"rc\": %d, \"status\": %d", r.rc, r.status);
        if (r.rc == LINREC_OK) {
            printf(", \"ms_median\": %.5f, \"ms_min\": %.5f, \"gbps_median\": %.1f, \"gbps_best\": %.1f, \"gelem_s\": %.2f",
                   r.ms_med, r.ms_min, bytes / (r.ms_med * 1e6), bytes / (r.ms_min * 1e6), elems / (r.ms_med * 1e6));
            if (a.verify) {
                printf(", \"max_abs_err\": [%g, %g], \"out_of_tol\": [%llu, %llu]", r.max_err0, r.max_err1, r.bad0, r.bad1);
                if (r.bad0 || r.bad1) worst = 3;
            }
            if (r.status != LINREC_OK) worst = 4;
        } else {
            printf(", \"error\": \"%s\"", linrec_b200_strerror(r.rc));
            if (!a.sweep) worst = 5;
        }
        printf("}\n");
        fflush(stdout);
    }
    if (!a.dump.empty()) {
        CK(cudaDeviceSynchronize());
        std::vector<T> host(total);
        auto put = [&](const char* what, const T* dev) {
            if (!dev) return;
            CK(cudaMemcpy(host.data(), dev, total * sizeof(T), cudaMemcpyDeviceToHost));
            const std::string path = a.dump + "." + what + ".bin";
            FILE* f = fopen(path.c_str(), "wb");
            if (!f || fwrite(host.data(), sizeof(T), total, f) != total) {
                fprintf(stderr, "cannot write %s\n", path.c_str());
                worst = worst ? worst : 6;
            }
            if (f) fclose(f);
        };
        put("in0", in0);
        put("c", c);
        put("y", yfw);
        put("out0", out0);
        put("out1", out1);
    }
    cudaFree(in0); cudaFree(c); cudaFree(out0); cudaFree(ref0); cudaFree(ws); cudaFree(d_max); cudaFree(d_bad);
    if (yfw) cudaFree(yfw);
    if (out1) cudaFree(out1);
    if (ref1) cudaFree(ref1);
    if (flush_buf) cudaFree(flush_buf);
    return worst;
}

int main(int argc, char** argv)
{
    Args a;
    for (int i = 1; i < argc; ++i) {
        std::string s = argv[i];
        auto next = [&]() -> const char* {
            if (i + 1 >= argc) { usage(); exit(1); }
            return argv[++i];
        };
        if (s == "--numseq") a.numseq = atoll(next());
        else if (s == "--seqlen") a.seqlen = atoll(next());
        else if (s == "--stride") a.stride = atoll(next());
        else if (s == "--chan") a.chan = atoll(next());
        else if (s == "--reverse") a.reverse = 1;
        else if (s == "--bwd") a.bwd = 1;
        else if (s == "--dtype") { std::string d = next(); a.dtype = d == "bf16" ? LINREC_DTYPE_BF16 : d == "f16" ? LINREC_DTYPE_F16 : LINREC_DTYPE_F32; }
        else if (s == "--clo") a.clo = (float)atof(next());
        else if (s == "--chi") a.chi = (float)atof(next());
        else if (s == "--iters") a.iters = atoi(next());
        else if (s == "--warmup") a.warmup = atoi(next());
        else if (s == "--flush") a.flush = 1;
        else if (s == "--sweep") a.sweep = 1;
        else if (s == "--no-verify") a.verify = 0;
        else if (s == "--dump") a.dump = next();
        else if (s == "--kind") {
            std::string k = next();
            a.kind = k == "ref" ? LINREC_KIND_REF : k == "tile" ? LINREC_KIND_TILE : LINREC_KIND_PIPE;
        } else if (s == "--opt") {
            std::string kv = next();
            const size_t eq = kv.find('=');
            if (eq == std::string::npos) { usage(); return 1; }
            a.opt_names.push_back(kv.substr(0, eq));
            a.opt_values.push_back(atoi(kv.c_str() + eq + 1));
        } else {
            usage();
            return 1;
        }
    }
    if (a.stride <= 0) a.stride = a.seqlen;
    if (a.iters < 1) a.iters = 1;
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, 0));
    fprintf(stderr, "# device: %s, %d SMs, library version %d\n", prop.name, prop.multiProcessorCount, linrec_b200_version());
    return a.dtype == LINREC_DTYPE_F32 ? run<float>(a) : a.dtype == LINREC_DTYPE_BF16 ? run<__nv_bfloat16>(a) : run<__half>(a);
}
