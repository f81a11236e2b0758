// Bulk-copy kernel variants: 256-thread tiles and the three-slot 128-thread ring.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_tma_variants_0(std::vector<TmaVariant>& v)
{
    v.push_back(make_tma_variant<16, 256, 2, 1>());
    v.push_back(make_tma_variant<16, 256, 3, 1>());
    v.push_back(make_tma_variant<16, 128, 3, 1>());
    v.push_back(make_tma_variant<16, 128, 2, 1>());
}

}  // namespace linrec_variants
