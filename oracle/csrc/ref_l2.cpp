// Exposes the reference's own portable L2 distance code (compiled from its source file, which
// is found on the include path given at build time; nothing of it is copied here).
#include "l2distance.codelet.cpp"

extern "C" float ref_l2dist(const float* a, const float* b, size_t n) { return l2dist<float>(a, b, n); }
extern "C" float ref_l2distgrad(float a, const float* b, const float* dist, const float* grad, size_t n) {
    return l2distgrad<float>(a, b, dist, grad, n);
}
