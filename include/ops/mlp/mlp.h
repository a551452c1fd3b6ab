/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/mlp/mlp.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
