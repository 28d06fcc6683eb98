// nz::data::Dimension: the {N, C, H, W} shape of a tensor with contiguous NCHW strides and
// NeuZephyr's broadcast rule (N and C may broadcast; H and W must agree). Mirrors
// include/NeuZephyr/Dimension.cuh / src/Dimension.cu of the reference.
#pragma once
#include <array>
#include <cstddef>
#include <ostream>
#include <stdexcept>
#include <vector>

namespace nz::data {

class Dimension {
public:
    Dimension() : d_{1, 1, 1, 1} {}
    Dimension(size_t n, size_t c, size_t h, size_t w) : d_{n, c, h, w} {}
    Dimension(const std::vector<size_t>& v) {  // NOLINT: implicit, as in the reference
        if (v.size() != 4) throw std::invalid_argument("Dimension needs 4 extents");
        d_ = {v[0], v[1], v[2], v[3]};
    }

    size_t N() const { return d_[0]; }
    size_t C() const { return d_[1]; }
    size_t H() const { return d_[2]; }
    size_t W() const { return d_[3]; }
    size_t size() const { return d_[0] * d_[1] * d_[2] * d_[3]; }
    size_t operator[](size_t i) const { return d_.at(i); }
    size_t& operator[](size_t i) { return d_.at(i); }
    // contiguous strides {C*H*W, H*W, W, 1}
    size_t getStride(size_t i) const {
        switch (i) {
            case 0: return d_[1] * d_[2] * d_[3];
            case 1: return d_[2] * d_[3];
            case 2: return d_[3];
            case 3: return 1;
            default: throw std::out_of_range("stride index");
        }
    }
    std::array<size_t, 4> getDims() const { return d_; }
    bool operator==(const Dimension& o) const { return d_ == o.d_; }
    bool operator!=(const Dimension& o) const { return !(*this == o); }
    // N and C are compatible if equal or one of them is 1
    bool isBroadcastCompatible(const Dimension& o) const {
        for (int i = 0; i < 2; i++)
            if (d_[i] != o.d_[i] && d_[i] != 1 && o.d_[i] != 1) return false;
        return true;
    }
    Dimension Broadcast(const Dimension& o) const {
        if (!isBroadcastCompatible(o)) throw std::invalid_argument("Shapes are not broadcast compatible.");
        return Dimension(d_[0] > o.d_[0] ? d_[0] : o.d_[0], d_[1] > o.d_[1] ? d_[1] : o.d_[1], d_[2], d_[3]);
    }
    void reshape(size_t n, size_t c, size_t h, size_t w) {
        if (n * c * h * w != size()) throw std::invalid_argument("reshape changes the element count");
        d_ = {n, c, h, w};
    }

private:
    std::array<size_t, 4> d_;
};

inline std::ostream& operator<<(std::ostream& os, const Dimension& d) {
    return os << "(" << d.N() << ", " << d.C() << ", " << d.H() << ", " << d.W() << ")";
}

}  // namespace nz::data
