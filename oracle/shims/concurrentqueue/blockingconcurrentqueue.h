// Test infrastructure (oracle build only): blocking variant of the queue in
// concurrentqueue.h, used by the reference scheduler to wait for ready nodes.
#pragma once
#include <condition_variable>
#include <cstddef>
#include <deque>
#include <mutex>
#include <utility>

namespace moodycamel {

template <class T>
class BlockingConcurrentQueue {
    mutable std::mutex      mutex_;
    std::condition_variable ready_;
    std::deque<T>           items_;

public:
    BlockingConcurrentQueue() = default;

    bool enqueue(const T &item) {
        { std::lock_guard<std::mutex> g(mutex_); items_.push_back(item); }
        ready_.notify_one();
        return true;
    }
    bool enqueue(T &&item) {
        { std::lock_guard<std::mutex> g(mutex_); items_.push_back(std::move(item)); }
        ready_.notify_one();
        return true;
    }

    bool try_dequeue(T &out) {
        std::lock_guard<std::mutex> g(mutex_);
        if (items_.empty()) { return false; }
        out = std::move(items_.front());
        items_.pop_front();
        return true;
    }

    void wait_dequeue(T &out) {
        std::unique_lock<std::mutex> g(mutex_);
        ready_.wait(g, [this] { return !items_.empty(); });
        out = std::move(items_.front());
        items_.pop_front();
    }

    std::size_t size_approx() const { std::lock_guard<std::mutex> g(mutex_); return items_.size(); }
};

}  // namespace moodycamel
