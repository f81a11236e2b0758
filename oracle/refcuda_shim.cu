// TEST INFRASTRUCTURE ONLY -- C entry points around the reference's own sequential CUDA kernels.
//
// The kernels come from the reference tree (linrec/impl/cuda/linrec_ref.cuh, found through the
// include path given by oracle/build.py); this file only launches them the way the reference's
// host code does (linrec/impl/cuda/linrec_ref.cu:33-42 and :85): one block per row, one thread
// per block, on the caller's stream.  The result is a GPU-side checker for the parity tests.
//
// Known defect of the reference that this shim has to live with: with rev=true the backward
// kernel's d_coeffs loop runs two elements past the row (linrec/impl/cuda/linrec_ref.cuh:90).
// It reads outputs[L], outputs[L+1], d_inputs[L] and writes d_coeffs[L] of every row, i.e. it
// touches the head of the next row and, for the last row, memory after the tensor.  To keep
// every access inside an allocation the reverse backward is run on private copies that carry
// two extra floats of slack; the value it leaves in d_coeffs[r][0] for r >= 1 is decided by a
// race between blocks r-1 and r, so callers must not compare that column.
#include <cuda_runtime.h>
#include <stdint.h>

#include <linrec_ref.cuh>

#define SHIM_API extern "C" __attribute__((visibility("default")))

SHIM_API int refcuda_fwd_f32(const float* x, const float* c, float* y, int numseq, int seqlen,
                             int reverse, void* stream)
{
    if (numseq <= 0 || seqlen <= 0) return 0;
    if ((int64_t)numseq * seqlen > 2147483647LL) return -1;   // the kernels index with int
    linrec_ref_fwd_kernel<float><<<numseq, 1, 0, (cudaStream_t)stream>>>(x, c, y, seqlen, reverse != 0);
    return (int)cudaGetLastError();
}

SHIM_API int refcuda_bwd_f32(const float* dy, const float* c, const float* y, float* dx, float* dc,
                             int numseq, int seqlen, int reverse, void* stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (numseq <= 0 || seqlen <= 0) return 0;
    const int64_t n = (int64_t)numseq * seqlen;
    if (n + 2 > 2147483647LL) return -1;
    if (!reverse) {
        linrec_ref_bwd_kernel<float><<<numseq, 1, 0, stream>>>(dy, c, y, dx, dc, seqlen, false);
        return (int)cudaGetLastError();
    }
    // reverse: padded private copies (see the note at the top of this file)
    float *yp = nullptr, *dxp = nullptr, *dcp = nullptr;
    const size_t bytes = (size_t)(n + 2) * sizeof(float);
    cudaError_t e;
    if ((e = cudaMalloc(&yp, bytes)) != cudaSuccess) return (int)e;
    if ((e = cudaMalloc(&dxp, bytes)) != cudaSuccess) { cudaFree(yp); return (int)e; }
    if ((e = cudaMalloc(&dcp, bytes)) != cudaSuccess) { cudaFree(yp); cudaFree(dxp); return (int)e; }
    cudaMemsetAsync(yp, 0, bytes, stream);
    cudaMemsetAsync(dxp, 0, bytes, stream);
    cudaMemsetAsync(dcp, 0, bytes, stream);
    cudaMemcpyAsync(yp, y, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, stream);
    linrec_ref_bwd_kernel<float><<<numseq, 1, 0, stream>>>(dy, c, yp, dxp, dcp, seqlen, true);
    e = cudaGetLastError();
    cudaMemcpyAsync(dx, dxp, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, stream);
    cudaMemcpyAsync(dc, dcp, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, stream);
    cudaStreamSynchronize(stream);
    cudaFree(yp); cudaFree(dxp); cudaFree(dcp);
    return (int)e;
}
