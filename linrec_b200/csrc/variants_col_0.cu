// Middle-axis kernel variants: 128-thread tiles.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_col_variants_0(std::vector<ColVariant>& v)
{
    v.push_back(make_col_variant<128, 32, 3>());
    v.push_back(make_col_variant<128, 32, 2>());
    v.push_back(make_col_variant<128, 32, 4>());
    v.push_back(make_col_variant<256, 32, 2>());
}

}  // namespace linrec_variants
