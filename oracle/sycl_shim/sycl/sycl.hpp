// Host-only stand-in for the handful of SYCL names that the reference's
// per-group helper header (src/csrc/kernels/internal/quant_tile.hpp) uses, so
// that header can be compiled by g++ where it lies and run on the CPU as a
// checker.  TEST INFRASTRUCTURE ONLY: nothing shipped includes this file.
//
// Semantics follow the SYCL 2020 specification: sycl::round rounds halfway
// cases away from zero (std::round), fmin/fmax ignore a NaN operand
// (std::fmin/std::fmax), clamp is min(max(x, lo), hi), vec<float,4>::load and
// ::store move four consecutive elements at element offset 4*offset.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>

namespace sycl {

template <typename T>
class global_ptr {
public:
    explicit global_ptr(T* p) : p_(p) {}
    T* get() const { return p_; }
private:
    T* p_;
};

template <typename T, int N>
class vec {
public:
    T& operator[](int i) { return v_[i]; }
    const T& operator[](int i) const { return v_[i]; }
    void load(std::size_t offset, global_ptr<const T> p) {
        for (int i = 0; i < N; ++i) v_[i] = p.get()[offset * N + i];
    }
    void store(std::size_t offset, global_ptr<T> p) const {
        for (int i = 0; i < N; ++i) p.get()[offset * N + i] = v_[i];
    }
private:
    T v_[N];
};

inline float fmin(float a, float b) { return std::fmin(a, b); }
inline float fmax(float a, float b) { return std::fmax(a, b); }
inline float round(float a) { return std::round(a); }
inline int clamp(int x, int lo, int hi) { return std::min(std::max(x, lo), hi); }

}  // namespace sycl
