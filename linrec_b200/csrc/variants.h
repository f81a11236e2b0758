// The compiled kernel variants: one table row per (elements per thread, threads, ring depth, ...)
// with the kernel entry points for every storage type, pass and direction.  The rows are built in
// several translation units (variants_*.cu) so that the kernels compile in parallel; capi.cu puts the
// tables together.  Counterpart of CONFIG_LIST and the compile-time dispatch of the reference
// (linrec/impl/cuda/linrec.h:8-13, dispatch.h:53-108).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <vector>

#include "scan_kernels.cuh"
#include "column_kernels.cuh"

namespace linrec_variants {

using linrec::ScanParams;

using TmaFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                       const CUtensorMap, const ScanParams);
using GenericFn = void (*)(const ScanParams);

struct TmaVariant {
    int E, NT, S, OB;
    size_t smem[3][2];      // [dtype][bwd]
    TmaFn fn[3][2][2];      // [dtype][bwd][asc]
};

template <int E, int NT, int S, int OB>
TmaVariant make_tma_variant()
{
    using namespace linrec;
    TmaVariant v{};
    v.E = E; v.NT = NT; v.S = S; v.OB = OB;
    v.smem[0][0] = TmaLayout<float, E, NT, S, OB, false>::kDynSmem;
    v.smem[0][1] = TmaLayout<float, E, NT, S, OB, true>::kDynSmem;
    v.smem[1][0] = TmaLayout<__nv_bfloat16, E, NT, S, OB, false>::kDynSmem;
    v.smem[1][1] = TmaLayout<__nv_bfloat16, E, NT, S, OB, true>::kDynSmem;
    v.fn[0][0][0] = linrec_tma_kernel<float, E, NT, S, OB, false, false>;
    v.fn[0][0][1] = linrec_tma_kernel<float, E, NT, S, OB, false, true>;
    v.fn[0][1][0] = linrec_tma_kernel<float, E, NT, S, OB, true, false>;
    v.fn[0][1][1] = linrec_tma_kernel<float, E, NT, S, OB, true, true>;
    v.fn[1][0][0] = linrec_tma_kernel<__nv_bfloat16, E, NT, S, OB, false, false>;
    v.fn[1][0][1] = linrec_tma_kernel<__nv_bfloat16, E, NT, S, OB, false, true>;
    v.fn[1][1][0] = linrec_tma_kernel<__nv_bfloat16, E, NT, S, OB, true, false>;
    v.fn[1][1][1] = linrec_tma_kernel<__nv_bfloat16, E, NT, S, OB, true, true>;
    v.smem[2][0] = TmaLayout<__half, E, NT, S, OB, false>::kDynSmem;
    v.smem[2][1] = TmaLayout<__half, E, NT, S, OB, true>::kDynSmem;
    v.fn[2][0][0] = linrec_tma_kernel<__half, E, NT, S, OB, false, false>;
    v.fn[2][0][1] = linrec_tma_kernel<__half, E, NT, S, OB, false, true>;
    v.fn[2][1][0] = linrec_tma_kernel<__half, E, NT, S, OB, true, false>;
    v.fn[2][1][1] = linrec_tma_kernel<__half, E, NT, S, OB, true, true>;
    return v;
}

struct GenericVariant {
    int E, NT, S;
    size_t smem[3][2];      // [dtype][bwd]: dynamic shared memory (0 for the plain-load kernel)
    GenericFn fn[3][2][2];  // [dtype][bwd][asc]
};

template <int E, int NT>
GenericVariant make_generic_variant()
{
    using namespace linrec;
    GenericVariant v{};
    v.E = E; v.NT = NT; v.S = 1;
    v.fn[0][0][0] = linrec_generic_kernel<float, E, NT, false, false>;
    v.fn[0][0][1] = linrec_generic_kernel<float, E, NT, false, true>;
    v.fn[0][1][0] = linrec_generic_kernel<float, E, NT, true, false>;
    v.fn[0][1][1] = linrec_generic_kernel<float, E, NT, true, true>;
    v.fn[1][0][0] = linrec_generic_kernel<__nv_bfloat16, E, NT, false, false>;
    v.fn[1][0][1] = linrec_generic_kernel<__nv_bfloat16, E, NT, false, true>;
    v.fn[1][1][0] = linrec_generic_kernel<__nv_bfloat16, E, NT, true, false>;
    v.fn[1][1][1] = linrec_generic_kernel<__nv_bfloat16, E, NT, true, true>;
    v.fn[2][0][0] = linrec_generic_kernel<__half, E, NT, false, false>;
    v.fn[2][0][1] = linrec_generic_kernel<__half, E, NT, false, true>;
    v.fn[2][1][0] = linrec_generic_kernel<__half, E, NT, true, false>;
    v.fn[2][1][1] = linrec_generic_kernel<__half, E, NT, true, true>;
    return v;
}

template <int E, int NT, int S, int CB>
GenericVariant make_async_variant()
{
    using namespace linrec;
    GenericVariant v{};
    v.E = E; v.NT = NT; v.S = S;
    v.smem[0][0] = AsyncLayout<float, E, NT, S, false>::kDynSmem;
    v.smem[0][1] = AsyncLayout<float, E, NT, S, true>::kDynSmem;
    v.smem[1][0] = AsyncLayout<__nv_bfloat16, E, NT, S, false>::kDynSmem;
    v.smem[1][1] = AsyncLayout<__nv_bfloat16, E, NT, S, true>::kDynSmem;
    v.smem[2][0] = AsyncLayout<__half, E, NT, S, false>::kDynSmem;
    v.smem[2][1] = AsyncLayout<__half, E, NT, S, true>::kDynSmem;
    v.fn[0][0][0] = linrec_async_kernel<float, E, NT, S, CB, false, false>;
    v.fn[0][0][1] = linrec_async_kernel<float, E, NT, S, CB, false, true>;
    v.fn[0][1][0] = linrec_async_kernel<float, E, NT, S, CB, true, false>;
    v.fn[0][1][1] = linrec_async_kernel<float, E, NT, S, CB, true, true>;
    v.fn[1][0][0] = linrec_async_kernel<__nv_bfloat16, E, NT, S, CB, false, false>;
    v.fn[1][0][1] = linrec_async_kernel<__nv_bfloat16, E, NT, S, CB, false, true>;
    v.fn[1][1][0] = linrec_async_kernel<__nv_bfloat16, E, NT, S, CB, true, false>;
    v.fn[1][1][1] = linrec_async_kernel<__nv_bfloat16, E, NT, S, CB, true, true>;
    v.fn[2][0][0] = linrec_async_kernel<__half, E, NT, S, CB, false, false>;
    v.fn[2][0][1] = linrec_async_kernel<__half, E, NT, S, CB, false, true>;
    v.fn[2][1][0] = linrec_async_kernel<__half, E, NT, S, CB, true, false>;
    v.fn[2][1][1] = linrec_async_kernel<__half, E, NT, S, CB, true, true>;
    return v;
}

using ColFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                       const CUtensorMap, const linrec::ColParams);
struct ColVariant {
    int NT, LC, S;
    size_t smem[3][2];     // [dtype][bwd]
    ColFn fn[3][2][2];     // [dtype][bwd][asc]; null where the variant does not exist for the type
};

template <typename ST, int NT, int LC, int S>
void fill_col_variant(ColVariant& v, int di)
{
    using namespace linrec;
    if constexpr (NT * (4 / (int)sizeof(ST)) <= 256) {
        v.smem[di][0] = ColLayout<ST, NT, LC, S, false>::kDynSmem;
        v.smem[di][1] = ColLayout<ST, NT, LC, S, true>::kDynSmem;
        v.fn[di][0][0] = linrec_column_kernel<ST, NT, LC, S, false, false>;
        v.fn[di][0][1] = linrec_column_kernel<ST, NT, LC, S, false, true>;
        v.fn[di][1][0] = linrec_column_kernel<ST, NT, LC, S, true, false>;
        v.fn[di][1][1] = linrec_column_kernel<ST, NT, LC, S, true, true>;
    }
}

template <int NT, int LC, int S>
ColVariant make_col_variant()
{
    ColVariant v{};
    v.NT = NT; v.LC = LC; v.S = S;
    fill_col_variant<float, NT, LC, S>(v, 0);
    fill_col_variant<__nv_bfloat16, NT, LC, S>(v, 1);
    fill_col_variant<__half, NT, LC, S>(v, 2);
    return v;
}


// Filled by the variants_*.cu translation units.
void add_tma_variants_0(std::vector<TmaVariant>& v);
void add_tma_variants_1(std::vector<TmaVariant>& v);
void add_tma_variants_2(std::vector<TmaVariant>& v);
void add_async_variants(std::vector<GenericVariant>& v);
void add_word_variants(std::vector<GenericVariant>& v);
void add_col_variants_0(std::vector<ColVariant>& v);
void add_col_variants_1(std::vector<ColVariant>& v);

}  // namespace linrec_variants
