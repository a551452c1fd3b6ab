/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/matmul/matmul.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
