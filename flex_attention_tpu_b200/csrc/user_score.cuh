// The user score function the kernels call when they are instantiated with FLEXATTN_SCORE_USER.  This file is the
// placeholder of ahead-of-time builds (which never instantiate that score kind): a run-time compilation replaces
// it with a header of the same name generated from the registered expressions.
#pragma once

namespace flexattn {

// t = f(s, b, h, i, j): s = sm_scale * <q_i, k_j>, natural units
__device__ __forceinline__ float user_score(float s, int b, int h, int i, int j) { return s; }
// df / ds at the same point
__device__ __forceinline__ float user_dscore(float s, int b, int h, int i, int j) { return 1.0f; }

}  // namespace flexattn
