// Exposes the reference's own portable L1 distance code (compiled from its source file, which
// is found on the include path given at build time; nothing of it is copied here).
#include "l1distance.codelet.cpp"

extern "C" float ref_l1dist(const float* a, const float* b, size_t n) { return l1dist<float>(a, b, n); }
extern "C" float ref_l1distgrad(float a, const float* b, const float* grad, size_t n) {
    return l1distgrad<float>(a, b, grad, n);
}
