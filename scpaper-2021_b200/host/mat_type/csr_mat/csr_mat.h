// csr_mat under the reference's own include path (mat_type/csr_mat/csr_mat.h); every weight container of the
// path is defined in mat_type/mat_type.h.
#pragma once
#include "../mat_type.h"
