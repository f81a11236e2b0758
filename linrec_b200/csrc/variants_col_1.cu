// Middle-axis kernel variants: 64- and 32-thread tiles.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_col_variants_1(std::vector<ColVariant>& v)
{
    v.push_back(make_col_variant<64, 64, 3>());
    v.push_back(make_col_variant<64, 64, 2>());
    v.push_back(make_col_variant<32, 64, 3>());
    v.push_back(make_col_variant<32, 64, 2>());
    v.push_back(make_col_variant<32, 128, 2>());
}

}  // namespace linrec_variants
