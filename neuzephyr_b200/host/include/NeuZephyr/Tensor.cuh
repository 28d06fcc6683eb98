// nz::data::Tensor: owning fp32 device buffer with an optional gradient buffer and a 4-D
// {N,C,H,W} shape (mirrors include/NeuZephyr/Tensor.cuh:134-1630, src/Tensor.cu). All work is
// asynchronous and ordered through StreamManager; host-visible results go through hostData()
// / sync().
#pragma once
#include <initializer_list>
#include <iterator>
#include <memory>
#include <ostream>
#include <stdexcept>
#include <vector>

#include "Dimension.cuh"
#include "StreamManager.cuh"

namespace nz::data {

class Tensor {
public:
    using size_type = size_t;
    using value_type = float;
    using shape_type = Dimension;

    Tensor();
    explicit Tensor(const shape_type& shape, bool requires_grad = false);
    // copies `data` (host memory when host == true, device memory otherwise)
    explicit Tensor(const shape_type& shape, value_type* data, bool requires_grad = false, bool host = true);
    explicit Tensor(const shape_type& shape, const std::initializer_list<value_type>& data,
                    bool requires_grad = false);
    Tensor(const Tensor& other);
    Tensor(Tensor&& other) noexcept;
    Tensor& operator=(const Tensor& other);
    Tensor& operator=(Tensor&& other) noexcept;
    ~Tensor();

    bool requiresGrad() const noexcept { return requires_grad_; }
    void setRequiresGrad(bool requires_grad);
    shape_type shape() const noexcept { return shape_; }
    size_type size() const noexcept { return size_; }
    value_type* data() const noexcept { return data_; }
    value_type* grad() const;
    std::vector<value_type> hostData() const noexcept;
    std::vector<value_type> hostGrad() const;

    void dataInject(value_type* data, bool grad = false) const;  // host pointer, size() values
    template <typename Iterator>
    void dataInject(Iterator begin, Iterator end, const bool grad = false) const {
        if (static_cast<size_type>(std::distance(begin, end)) < size_)
            throw std::runtime_error("The length of the input array is less than the size of the tensor.");
        std::vector<value_type> host(size_);
        auto it = begin;
        for (size_type i = 0; i < size_; ++i, ++it) host[i] = static_cast<value_type>(*it);
        dataInject(host.data(), grad);
    }
    void dataInject(const std::initializer_list<value_type>& data, bool grad = false) const;

    void zeroGrad() const;
    // A gradient buffer with exactly one consumer whose backward WRITES it (instead of adding to it) needs
    // no clearing: zeroGrad() skips it. Set by ComputeGraph for activations of fused models; the writing
    // node asks gradOverwritten() to choose between "=" and "+=". Results are the same either way.
    void setGradOverwritten(bool on) { grad_overwritten_ = on; }
    bool gradOverwritten() const noexcept { return grad_overwritten_; }
    // uniform (0, 1] from a 64-bit seed, as the reference's curand-based randomize in distribution
    // (src/Tensor.cu:298-300); the bit stream differs, so seeded comparisons inject data instead
    void randomize(unsigned long long seed = 0) const;
    void clear() const;
    void fill(value_type value, bool isGrad = false) const;
    void reshape(const shape_type& shape);

    void syncData() const;
    void syncGrad() const;
    void sync() const;

    // element-wise comparison with the reference's rule: |a-b| <= 1e-6 or relative <= 1e-5
    // (src/Tensor.cu:506-548); compares gradients too when both tensors require them
    bool operator==(const Tensor& other) const;
    bool operator!=(const Tensor& other) const { return !(*this == other); }
    // batched matrix product at fp32 accuracy with N / C broadcast (src/Tensor.cu:343-350): on the tensor
    // cores through a two-fp16 split of each operand, see tensorGeneralMatrixMul
    Tensor operator*(const Tensor& other) const;

    friend std::ostream& operator<<(std::ostream& os, const Tensor& t);

private:
    void allocate();
    void release();
    size_type size_ = 0;
    shape_type shape_;
    value_type* data_ = nullptr;
    value_type* grad_ = nullptr;
    bool requires_grad_ = false;
    bool grad_overwritten_ = false;
};

}  // namespace nz::data
