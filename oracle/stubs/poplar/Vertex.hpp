// Stand-in for the Poplar SDK header of the same name: the vertex field wrappers as plain
// views, so that the reference's codelet sources compile on the host.  Test infrastructure only.
#pragma once

#include <cstddef>

namespace poplar {

struct Vertex {};

enum class VectorLayout { ONE_PTR, SPAN };

template <class T, VectorLayout L, unsigned Align = 0>
struct Vector {
    const T* ptr = nullptr;
    std::size_t count = 0;
    const T& operator[](std::size_t i) const { return ptr[i]; }
    std::size_t size() const { return count; }
};

template <class T>
struct Input {
    T value{};
    const T& operator*() const { return value; }
    auto& operator[](std::size_t i) const { return value[i]; }
    std::size_t size() const { return value.size(); }
};

template <class T>
struct Output {
    T* ptr = nullptr;
    T& operator*() { return *ptr; }
};

}  // namespace poplar
