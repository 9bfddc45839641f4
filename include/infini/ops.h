// Public C++ entry header: `#include <infini/ops.h>` (include/infini/ops.h of the reference).
#ifndef INFINI_OPS_H_
#define INFINI_OPS_H_

#include "ops/gemm.h"
#include "ops/moe_siblings.h"
#include "ops/moe_small.h"
#include "ops/repack.h"
#include "ops/router.h"

#endif
