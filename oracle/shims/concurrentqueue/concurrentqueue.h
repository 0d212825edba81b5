// Test infrastructure (oracle build only): a mutex-backed multi-producer /
// multi-consumer queue offering the four calls the reference CPU backend makes
// on its task queue. Ordering and throughput do not affect the arithmetic.
#pragma once
#include <cstddef>
#include <deque>
#include <mutex>
#include <utility>

namespace moodycamel {

template <class T>
class ConcurrentQueue {
protected:
    mutable std::mutex mutex_;
    std::deque<T>      items_;

public:
    ConcurrentQueue() = default;

    bool enqueue(const T &item) { std::lock_guard<std::mutex> g(mutex_); items_.push_back(item); return true; }
    bool enqueue(T &&item)      { std::lock_guard<std::mutex> g(mutex_); items_.push_back(std::move(item)); return true; }

    template <class It>
    bool enqueue_bulk(It first, std::size_t count) {
        std::lock_guard<std::mutex> g(mutex_);
        for (std::size_t i = 0; i < count; ++i, ++first) { items_.push_back(*first); }
        return true;
    }

    bool try_dequeue(T &out) {
        std::lock_guard<std::mutex> g(mutex_);
        if (items_.empty()) { return false; }
        out = std::move(items_.front());
        items_.pop_front();
        return true;
    }

    std::size_t size_approx() const { std::lock_guard<std::mutex> g(mutex_); return items_.size(); }
};

}  // namespace moodycamel
