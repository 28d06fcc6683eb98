// nz::cuStrm::StreamManager<T>: the singleton stream scheduler of the host layer.
//
// Observable semantics kept from NeuZephyr (include/NeuZephyr/StreamManager.cuh:131-911,
// include/NeuZephyr/EventPool.cuh:165-457): a pool of 16 non-blocking streams handed out
// round-robin under a mutex; every operation first makes its stream wait on the pending
// events of the pointers it touches and afterwards records an event keyed by the pointers it
// wrote; syncData(ptr) blocks the host until a pointer has no pending work; sync() drains
// every stream; allocation and release do not block the host and are ordered with the work
// on the buffer.
// Deliberate differences: readers are tracked as well as writers (the reference orders a
// freeAsync only after writers, so a buffer can be released under a kernel still reading
// it); malloc takes a byte count and allocates exactly that (the reference multiplies by
// sizeof(T) a second time); events are retired by polling instead of one host callback per
// launch; released blocks go to a size-keyed cache owned by the manager instead of back
// to the driver (the reference calls cudaMallocAsync / cudaFreeAsync per tensor, whose pool,
// with buffers allocated and released on 16 rotating streams, re-maps memory every training
// step). A cached block keeps the pending events of its last owner, so whoever gets it next
// is ordered after that owner's kernels by the same per-pointer event mechanism.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <functional>
#include <initializer_list>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "NeuZephyrCudaErrorHandling.cuh"

namespace nz::cuStrm {

class EventPool {
public:
    explicit EventPool(size_t reserve = 128);
    ~EventPool();
    cudaEvent_t acquire();
    void release(cudaEvent_t e);

private:
    std::mutex mu_;
    std::vector<cudaEvent_t> free_;
};

template <typename T>
class StreamManager {
public:
    static StreamManager& Instance() {
        static StreamManager inst(16, 128);
        return inst;
    }
    StreamManager(const StreamManager&) = delete;
    StreamManager& operator=(const StreamManager&) = delete;
    ~StreamManager();

    cudaStream_t getStream();
    size_t streamCount() const { return streams_.size(); }

    // make `stream` wait for the pending writers (and, for a pointer about to be written,
    // also the pending readers) of `ptr`
    void streamWait(const void* ptr, cudaStream_t stream, bool will_write = false);
    void recordData(const void* ptr, cudaStream_t stream);  // ptr was written on stream
    void recordRead(const void* ptr, cudaStream_t stream);  // ptr was read on stream
    void syncData(const void* ptr);                         // host waits until ptr is idle
    void sync();                                            // host waits for every stream

    // One operation: pick a stream, order it after the operands' pending work, run
    // `launch(stream)`, publish events. Returns the stream used.
    cudaStream_t run(std::initializer_list<const void*> writes, std::initializer_list<const void*> reads,
                     const std::function<void(cudaStream_t)>& launch);

    // stream-ordered memory
    void malloc(T** ptr, size_t bytes);
    void free(T* ptr);
    void freeAsync(T* ptr) { free(ptr); }
    void memset(T* ptr, int value, size_t bytes);
    void memcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind);

    // scratch for library calls: valid until released; stream-ordered on `stream`
    void* scratch(size_t bytes, cudaStream_t stream);
    void releaseScratch(void* p, cudaStream_t stream);

    // hands every cached block back to the driver (after draining all streams)
    void trim();
    size_t cachedBytes();

private:
    StreamManager(size_t n_streams, size_t n_events);
    struct Pending {
        std::vector<cudaEvent_t> writers, readers;
    };
    void prune(Pending& p);
    void waitAll(const std::vector<cudaEvent_t>& v, cudaStream_t stream);

    std::vector<cudaStream_t> streams_;
    size_t next_ = 0;
    std::mutex mu_;
    std::unordered_map<const void*, Pending> pending_;
    EventPool events_;

    void* allocBlock(size_t bytes);
    void releaseBlock(void* p);
    std::multimap<size_t, void*> cache_;         // free blocks by size
    std::unordered_map<void*, size_t> live_;     // blocks handed out
    size_t cached_bytes_ = 0;
};

extern template class StreamManager<float>;

}  // namespace nz::cuStrm
