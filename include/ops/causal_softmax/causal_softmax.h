/* Path-compatible entry: C callers of the reference include this path
 * (reference include/ops/causal_softmax/causal_softmax.h); all declarations live in infiniop.h. */
#include "../../infiniop.h"
