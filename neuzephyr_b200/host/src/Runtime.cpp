// StreamManager / EventPool / Tensor of the host layer.
#include <NeuZephyr/StreamManager.cuh>
#include <NeuZephyr/Tensor.cuh>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <random>

namespace nz::cuStrm {

EventPool::EventPool(size_t) {}
EventPool::~EventPool() {
    for (auto e : free_) cudaEventDestroy(e);
}
cudaEvent_t EventPool::acquire() {
    std::lock_guard<std::mutex> lk(mu_);
    if (!free_.empty()) {
        cudaEvent_t e = free_.back();
        free_.pop_back();
        return e;
    }
    cudaEvent_t e;
    CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
}
void EventPool::release(cudaEvent_t e) {
    std::lock_guard<std::mutex> lk(mu_);
    free_.push_back(e);
}

template <typename T>
StreamManager<T>::StreamManager(size_t n_streams, size_t n_events) : events_(n_events) {
    streams_.resize(n_streams);
    for (auto& s : streams_) CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
}
template <typename T>
StreamManager<T>::~StreamManager() {
    for (auto s : streams_) cudaStreamSynchronize(s);
    for (auto& kv : cache_) cudaFree(kv.second);
    for (auto s : streams_) cudaStreamDestroy(s);
}
template <typename T>
cudaStream_t StreamManager<T>::getStream() {
    std::lock_guard<std::mutex> lk(mu_);
    cudaStream_t s = streams_[next_];
    next_ = (next_ + 1) % streams_.size();
    return s;
}
template <typename T>
void StreamManager<T>::prune(Pending& p) {
    auto done = [this](cudaEvent_t e) {
        if (cudaEventQuery(e) == cudaSuccess) {
            events_.release(e);
            return true;
        }
        return false;
    };
    p.writers.erase(std::remove_if(p.writers.begin(), p.writers.end(), done), p.writers.end());
    p.readers.erase(std::remove_if(p.readers.begin(), p.readers.end(), done), p.readers.end());
}
template <typename T>
void StreamManager<T>::waitAll(const std::vector<cudaEvent_t>& v, cudaStream_t stream) {
    for (auto e : v) CHECK(cudaStreamWaitEvent(stream, e, 0));
}
template <typename T>
void StreamManager<T>::streamWait(const void* ptr, cudaStream_t stream, bool will_write) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lk(mu_);
    auto it = pending_.find(ptr);
    if (it == pending_.end()) return;
    prune(it->second);
    waitAll(it->second.writers, stream);
    if (will_write) waitAll(it->second.readers, stream);
    if (it->second.writers.empty() && it->second.readers.empty()) pending_.erase(it);
}
template <typename T>
void StreamManager<T>::recordData(const void* ptr, cudaStream_t stream) {
    if (!ptr) return;
    cudaEvent_t e = events_.acquire();
    CHECK(cudaEventRecord(e, stream));
    std::lock_guard<std::mutex> lk(mu_);
    Pending& p = pending_[ptr];
    // everything recorded earlier was waited on by this stream: the new writer supersedes it
    for (auto o : p.writers) events_.release(o);
    for (auto o : p.readers) events_.release(o);
    p.writers.clear();
    p.readers.clear();
    p.writers.push_back(e);
}
template <typename T>
void StreamManager<T>::recordRead(const void* ptr, cudaStream_t stream) {
    if (!ptr) return;
    cudaEvent_t e = events_.acquire();
    CHECK(cudaEventRecord(e, stream));
    std::lock_guard<std::mutex> lk(mu_);
    Pending& p = pending_[ptr];
    if (p.readers.size() > 32) prune(p);
    p.readers.push_back(e);
}
template <typename T>
void StreamManager<T>::syncData(const void* ptr) {
    std::vector<cudaEvent_t> ev;
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = pending_.find(ptr);
        if (it == pending_.end()) return;
        ev = it->second.writers;
        ev.insert(ev.end(), it->second.readers.begin(), it->second.readers.end());
    }
    for (auto e : ev) CHECK(cudaEventSynchronize(e));
}
template <typename T>
void StreamManager<T>::sync() {
    for (auto s : streams_) CHECK(cudaStreamSynchronize(s));
}
template <typename T>
cudaStream_t StreamManager<T>::run(std::initializer_list<const void*> writes,
                                   std::initializer_list<const void*> reads,
                                   const std::function<void(cudaStream_t)>& launch) {
    cudaStream_t s = getStream();
    for (auto p : reads) streamWait(p, s, false);
    for (auto p : writes) streamWait(p, s, true);
    launch(s);
    for (auto p : reads) {
        bool also_written = false;
        for (auto w : writes) also_written |= (w == p);
        if (!also_written) recordRead(p, s);
    }
    for (auto p : writes) recordData(p, s);
    return s;
}
template <typename T>
void* StreamManager<T>::allocBlock(size_t bytes) {
    bytes = (std::max<size_t>(bytes, 1) + 511) / 512 * 512;
    // a cached block may be somewhat larger than asked: up to 2x for small ones, 1/8 over for large
    const size_t limit = bytes < (size_t(1) << 20) ? 2 * bytes : bytes + bytes / 8;
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = cache_.lower_bound(bytes);
        if (it != cache_.end() && it->first <= limit) {
            void* p = it->second;
            live_[p] = it->first;
            cached_bytes_ -= it->first;
            cache_.erase(it);
            return p;
        }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        trim();
        e = cudaMalloc(&p, bytes);
    }
    CHECK(e);
    std::lock_guard<std::mutex> lk(mu_);
    live_[p] = bytes;
    return p;
}
template <typename T>
void StreamManager<T>::releaseBlock(void* p) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(p);
    if (it == live_.end()) return;  // not handed out by this manager
    cache_.emplace(it->second, p);
    cached_bytes_ += it->second;
    live_.erase(it);
    // the block's pending events stay in pending_: its next owner waits on them
}
template <typename T>
void StreamManager<T>::trim() {
    sync();
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : cache_) {
        auto it = pending_.find(kv.second);
        if (it != pending_.end()) {
            for (auto e : it->second.writers) events_.release(e);
            for (auto e : it->second.readers) events_.release(e);
            pending_.erase(it);
        }
        CHECK(cudaFree(kv.second));
    }
    cache_.clear();
    cached_bytes_ = 0;
}
template <typename T>
size_t StreamManager<T>::cachedBytes() {
    std::lock_guard<std::mutex> lk(mu_);
    return cached_bytes_;
}
template <typename T>
void StreamManager<T>::malloc(T** ptr, size_t bytes) {
    *ptr = static_cast<T*>(allocBlock(bytes));
}
template <typename T>
void StreamManager<T>::free(T* ptr) {
    if (ptr) releaseBlock(ptr);
}
template <typename T>
void StreamManager<T>::memset(T* ptr, int value, size_t bytes) {
    run({ptr}, {}, [&](cudaStream_t s) { CHECK(cudaMemsetAsync(ptr, value, bytes, s)); });
}
template <typename T>
void StreamManager<T>::memcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
    const bool dst_dev = kind == cudaMemcpyHostToDevice || kind == cudaMemcpyDeviceToDevice;
    const bool src_dev = kind == cudaMemcpyDeviceToHost || kind == cudaMemcpyDeviceToDevice;
    cudaStream_t s = getStream();
    if (src_dev) streamWait(src, s, false);
    if (dst_dev) streamWait(dst, s, true);
    CHECK(cudaMemcpyAsync(dst, src, bytes, kind, s));
    if (src_dev) recordRead(src, s);
    if (dst_dev) recordData(dst, s);
    // copies that touch pageable host memory must be complete when the call returns
    if (!dst_dev || !src_dev) CHECK(cudaStreamSynchronize(s));
}
template <typename T>
void* StreamManager<T>::scratch(size_t bytes, cudaStream_t stream) {
    void* p = allocBlock(bytes ? bytes : 256);
    streamWait(p, stream, true);  // after whatever the block's previous owner left pending
    return p;
}
template <typename T>
void StreamManager<T>::releaseScratch(void* p, cudaStream_t stream) {
    if (!p) return;
    recordData(p, stream);
    releaseBlock(p);
}

template class StreamManager<float>;

}  // namespace nz::cuStrm

namespace nz::data {

using SM = cuStrm::StreamManager<float>;

Tensor::Tensor() : size_(0), shape_(0, 0, 0, 0) {}

void Tensor::allocate() {
    SM::Instance().malloc(&data_, size_ * sizeof(value_type));
    if (requires_grad_) SM::Instance().malloc(&grad_, size_ * sizeof(value_type));
}
void Tensor::release() {
    if (data_) SM::Instance().free(data_);
    if (grad_) SM::Instance().free(grad_);
    data_ = grad_ = nullptr;
}

Tensor::Tensor(const shape_type& shape, bool requires_grad)
    : size_(shape.size()), shape_(shape), requires_grad_(requires_grad) {
    allocate();
}
Tensor::Tensor(const shape_type& shape, value_type* data, bool requires_grad, bool host)
    : size_(shape.size()), shape_(shape), requires_grad_(requires_grad) {
    allocate();
    SM::Instance().memcpy(data_, data, size_ * sizeof(value_type),
                          host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
}
Tensor::Tensor(const shape_type& shape, const std::initializer_list<value_type>& data, bool requires_grad)
    : size_(shape.size()), shape_(shape), requires_grad_(requires_grad) {
    if (data.size() < size_) throw std::invalid_argument("Initializer list size is less than the tensor size.");
    allocate();
    std::vector<value_type> host(data.begin(), data.begin() + size_);
    SM::Instance().memcpy(data_, host.data(), size_ * sizeof(value_type), cudaMemcpyHostToDevice);
}
Tensor::Tensor(const Tensor& o) : size_(o.size_), shape_(o.shape_), requires_grad_(o.requires_grad_) {
    allocate();
    SM::Instance().memcpy(data_, o.data_, size_ * sizeof(value_type), cudaMemcpyDeviceToDevice);
    if (requires_grad_) SM::Instance().memcpy(grad_, o.grad_, size_ * sizeof(value_type), cudaMemcpyDeviceToDevice);
}
Tensor::Tensor(Tensor&& o) noexcept
    : size_(o.size_), shape_(o.shape_), data_(o.data_), grad_(o.grad_), requires_grad_(o.requires_grad_) {
    o.data_ = o.grad_ = nullptr;
    o.size_ = 0;
}
Tensor& Tensor::operator=(const Tensor& o) {
    if (this != &o) {
        Tensor tmp(o);
        *this = std::move(tmp);
    }
    return *this;
}
Tensor& Tensor::operator=(Tensor&& o) noexcept {
    if (this != &o) {
        release();
        size_ = o.size_; shape_ = o.shape_; data_ = o.data_; grad_ = o.grad_; requires_grad_ = o.requires_grad_;
        o.data_ = o.grad_ = nullptr;
        o.size_ = 0;
    }
    return *this;
}
Tensor::~Tensor() {
    try {
        release();
    } catch (...) {
    }
}

void Tensor::setRequiresGrad(bool requires_grad) {
    if (requires_grad && !grad_) SM::Instance().malloc(&grad_, size_ * sizeof(value_type));
    if (!requires_grad && grad_) {
        SM::Instance().free(grad_);
        grad_ = nullptr;
    }
    requires_grad_ = requires_grad;
}
Tensor::value_type* Tensor::grad() const {
    if (!requires_grad_) throw std::runtime_error("Tensor does not require gradients");
    return grad_;
}
std::vector<Tensor::value_type> Tensor::hostData() const noexcept {
    std::vector<value_type> h(size_);
    if (size_) SM::Instance().memcpy(h.data(), data_, size_ * sizeof(value_type), cudaMemcpyDeviceToHost);
    return h;
}
std::vector<Tensor::value_type> Tensor::hostGrad() const {
    if (!requires_grad_) throw std::runtime_error("Tensor does not require gradients");
    std::vector<value_type> h(size_);
    if (size_) SM::Instance().memcpy(h.data(), grad_, size_ * sizeof(value_type), cudaMemcpyDeviceToHost);
    return h;
}
void Tensor::dataInject(value_type* data, bool grad) const {
    if (grad && !requires_grad_) throw std::runtime_error("Tensor does not require gradients");
    SM::Instance().memcpy(grad ? grad_ : data_, data, size_ * sizeof(value_type), cudaMemcpyHostToDevice);
}
void Tensor::dataInject(const std::initializer_list<value_type>& data, bool grad) const {
    dataInject(data.begin(), data.end(), grad);
}
void Tensor::zeroGrad() const {
    if (requires_grad_ && !grad_overwritten_) SM::Instance().memset(grad_, 0, size_ * sizeof(value_type));
}
void Tensor::randomize(unsigned long long seed) const {
    std::mt19937_64 gen(seed);
    std::vector<value_type> h(size_);
    for (auto& v : h) v = static_cast<value_type>(((gen() >> 40) + 1) * (1.0 / 16777216.0));  // (0, 1]
    SM::Instance().memcpy(data_, h.data(), size_ * sizeof(value_type), cudaMemcpyHostToDevice);
}
void Tensor::clear() const { SM::Instance().memset(data_, 0, size_ * sizeof(value_type)); }
void Tensor::fill(value_type value, bool isGrad) const {
    if (isGrad && !requires_grad_) throw std::runtime_error("Tensor does not require gradients");
    value_type* p = isGrad ? grad_ : data_;
    SM::Instance().run({p}, {}, [&](cudaStream_t s) { NZB_CHECK(nzb_fill(p, value, (int64_t)size_, s)); });
}
void Tensor::reshape(const shape_type& shape) {
    if (shape.size() != size_) throw std::invalid_argument("reshape changes the element count");
    shape_ = shape;
}
void Tensor::syncData() const { SM::Instance().syncData(data_); }
void Tensor::syncGrad() const {
    if (requires_grad_) SM::Instance().syncData(grad_);
}
void Tensor::sync() const {
    syncData();
    syncGrad();
}
bool Tensor::operator==(const Tensor& o) const {
    if (shape_ != o.shape_ || requires_grad_ != o.requires_grad_) return false;
    auto close = [](const std::vector<value_type>& a, const std::vector<value_type>& b) {
        for (size_t i = 0; i < a.size(); i++) {
            const double d = std::fabs((double)a[i] - (double)b[i]);
            const double m = std::max(std::fabs((double)a[i]), std::fabs((double)b[i]));
            if (!(d <= 1e-6 || d <= 1e-5 * m)) return false;
        }
        return true;
    };
    if (!close(hostData(), o.hostData())) return false;
    if (requires_grad_ && !close(hostGrad(), o.hostGrad())) return false;
    return true;
}
std::ostream& operator<<(std::ostream& os, const Tensor& t) {
    const auto h = t.hostData();
    const auto s = t.shape();
    size_t i = 0;
    for (size_t n = 0; n < s.N(); n++)
        for (size_t c = 0; c < s.C(); c++) {
            os << "n=" << n << " c=" << c << "\n";
            for (size_t r = 0; r < s.H(); r++) {
                os << " [";
                for (size_t w = 0; w < s.W(); w++) os << (w ? ", " : "") << h[i++];
                os << "]\n";
            }
        }
    return os;
}

}  // namespace nz::data
