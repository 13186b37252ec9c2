// The rank-r adapter products with fused multiply-adds: k_gemm_skinny.cu compiled
// a second time as see::k::fast, without -fmad=false.  Used by the engine (lazy
// coherence), where nothing observes whether a sum was rounded once or twice per
// term; the strict seam keeps the bit-exact build.
#define SEE_SKINNY_NAMESPACE fast
#include "k_gemm_skinny.cu"
