// Bulk-copy kernel variants: 32 elements per thread.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_tma_variants_2(std::vector<TmaVariant>& v)
{
    v.push_back(make_tma_variant<32, 128, 2, 1>());
    v.push_back(make_tma_variant<32, 128, 3, 1>());
    v.push_back(make_tma_variant<32, 256, 2, 1>());
    v.push_back(make_tma_variant<32, 512, 2, 1>());   // 2-byte storage only (a 4-byte tile of 16384 exceeds a copy box)
    v.push_back(make_tma_variant<32, 512, 1, 1>());
}

}  // namespace linrec_variants
