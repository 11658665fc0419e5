// Stand-in for the Poplar SDK header of the same name, just enough for the portable (non-IPU)
// branches of the reference's distance codelets to compile as plain C++ on the host.
// Test infrastructure only: `half` here is a float in disguise, not a 16-bit type.
#pragma once

struct half {
    float v;
    half() : v(0.f) {}
    half(float x) : v(x) {}
    half(double x) : v(static_cast<float>(x)) {}
    half(int x) : v(static_cast<float>(x)) {}
    operator float() const { return v; }
};
inline half operator-(half a, half b) { return half(a.v - b.v); }
inline half operator*(half a, half b) { return half(a.v * b.v); }
inline bool operator<(half a, half b) { return a.v < b.v; }
