// Bulk-copy kernel variants: 512-thread tiles and the one-slot rings.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_tma_variants_1(std::vector<TmaVariant>& v)
{
    v.push_back(make_tma_variant<16, 512, 2, 1>());
    v.push_back(make_tma_variant<16, 512, 1, 1>());
    v.push_back(make_tma_variant<16, 256, 1, 1>());
    v.push_back(make_tma_variant<16, 128, 1, 1>());
}

}  // namespace linrec_variants
