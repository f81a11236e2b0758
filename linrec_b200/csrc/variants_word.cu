// cp.async kernel variants with 4-byte chunks.
// One of the translation units the kernel variants are spread over (see variants.h).
#include "variants.h"

namespace linrec_variants {

void add_word_variants(std::vector<GenericVariant>& v)
{
    v.push_back(make_async_variant<16, 128, 2, 4>());
    v.push_back(make_async_variant<16, 256, 2, 4>());
    v.push_back(make_async_variant<16, 512, 2, 4>());
}

}  // namespace linrec_variants
