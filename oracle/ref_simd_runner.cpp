// ref_simd_runner.cpp -- drives the reference's generated AVX2 ("simd") kernels on all host cores.
//
// TEST INFRASTRUCTURE ONLY.  The kernels themselves are produced at build time by the reference's
// own generator (tools/mslgen.cpp) from its prebuilt kernel artefacts (kernels/prebuilt/*.metal,
// *.ir) and compiled in place; nothing of them is stored in this repository.  This file is the small
// stand-in for the reference's Windows-only worker pool (src/stream.cpp): a persistent std::thread
// pool that hands out chunks planned with the reference's "guided" rule -- chunk = remaining /
// (2 * threads), at least min_chunk, in multiples of 16 (src/stream.cpp:389-403,
// src/runtime.cpp:505-511) -- each chunk's arguments offset the way the reference's kquantChunk does
// (llm/llm_kernels.cpp:281-288).  Bypassed Windows-only pieces: the Booth ELF loader, the MASM
// System-V thunk, the VEH fault guard, the guard-page allocator and src/runtime.cpp.

#include <kernelcore/kernel_registry.hpp>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <immintrin.h>
#include <mutex>
#include <thread>
#include <vector>

// The generated simd entry points (what kc::NativeKernel::simd points at in the reference's build).
extern "C" void kc_ksimd_matvec_q4k_q8(const kc::LaunchArgs*);
extern "C" void kc_ksimd_matvec_q6k_q8(const kc::LaunchArgs*);
extern "C" void kc_ksimd_quantize_q8x4(const kc::LaunchArgs*);

namespace {

struct Chunk {
    int64_t begin, length;
};

std::vector<Chunk> guided(int64_t total, unsigned threads, int64_t min_chunk, int64_t align) {
    std::vector<Chunk> out;
    for (int64_t b = 0; b < total;) {
        int64_t per = (total - b) / (2 * int64_t(threads));
        if (per < min_chunk) per = min_chunk;
        per = (per + align - 1) / align * align;
        if (per > total - b) per = total - b;
        out.push_back({b, per});
        b += per;
    }
    return out;
}

class Pool {
public:
    explicit Pool(unsigned n) {
        for (unsigned i = 1; i < n; ++i) th_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> l(m_);
            stop_ = true;
            ++gen_;
        }
        cv_.notify_all();
        for (auto& t : th_) t.join();
    }
    unsigned size() const { return unsigned(th_.size()) + 1; }
    // Runs fn(i) for i in [0, n) on all threads (caller included); returns when all are done.
    template <class F>
    void run(size_t n, F&& fn) {
        job_ = [&](size_t i) { fn(i); };
        n_ = n;
        next_.store(0);
        pending_.store(int(th_.size()));
        {
            std::lock_guard<std::mutex> l(m_);
            ++gen_;
        }
        cv_.notify_all();
        work();
        while (pending_.load(std::memory_order_acquire) != 0) _mm_pause();
    }

private:
    void work() {
        for (size_t i; (i = next_.fetch_add(1)) < n_;) job_(i);
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> l(m_);
                cv_.wait(l, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
            }
            work();
            pending_.fetch_sub(1, std::memory_order_release);
        }
    }
    std::vector<std::thread> th_;
    std::mutex m_;
    std::condition_variable cv_;
    uint64_t gen_ = 0;
    bool stop_ = false;
    std::function<void(size_t)> job_;
    size_t n_ = 0;
    std::atomic<size_t> next_{0};
    std::atomic<int> pending_{0};
};

Pool* g_pool = nullptr;

}  // namespace

extern "C" {

// Creates (or resizes) the pool; threads == 0 -> hardware concurrency.  Returns the thread count.
int kcref_simd_threads(int threads) {
    unsigned n = threads > 0 ? unsigned(threads) : std::thread::hardware_concurrency();
    if (n == 0) n = 1;
    if (!g_pool || g_pool->size() != n) {
        delete g_pool;
        g_pool = new Pool(n);
    }
    return int(n);
}

// One chunked launch of the reference's matvec_q4k_q8 / matvec_q6k_q8 simd kernel on its own weight
// stream qw (llm::ref::repackQ4K / repackQ6K output).  dims = {rows, k}.
void kcref_simd_matvec(int q6, const int32_t* qw, const int32_t* xq, const float* xd, float* y, int rows, int k,
                       int min_chunk) {
    if (!g_pool) kcref_simd_threads(0);
    const int words = q6 ? 53 : 37, nsb = k / 256;
    const int dims[2] = {rows, k};
    const kc::NativeKernelFn kn = q6 ? kc_ksimd_matvec_q6k_q8 : kc_ksimd_matvec_q4k_q8;
    const std::vector<Chunk> chunks = guided(rows, g_pool->size(), min_chunk, 16);
    g_pool->run(chunks.size(), [&](size_t i) {
        const Chunk c = chunks[i];
        kc::LaunchArgs a;
        kc::ArgPacker pk(a);
        pk.ptr(qw + c.begin / 8 * nsb * words * 8).ptr(xq).ptr(xd).ptr(y + c.begin).ptr(dims);
        pk.finish(c.length);
        kn(&a);
    });
}

// quantize_q8x4 through the reference's simd kernel (single launch; 96-256 threads of work).
void kcref_simd_quantize_q8x4(const float* x, int32_t* xq, float* xd, int count) {
    kc::LaunchArgs a;
    kc::ArgPacker pk(a);
    pk.ptr(x).ptr(xq).ptr(xd);
    pk.finish(count);
    kc_ksimd_quantize_q8x4(&a);
}

}  // extern "C"
