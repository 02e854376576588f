// Stands at the include path of the reference header of the same name; everything on the ring-packed
// matrix-multiply path is declared in ckks_llm_compat.hpp.
#pragma once
#include "../../../../ckks_llm_compat.hpp"
