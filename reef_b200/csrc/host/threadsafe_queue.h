// Bounded mutex-guarded FIFO used for the real-time and best-effort task queues
// (reference: src/reef/util/threadsafe_queue.h:14-69, capacity 10000).
#pragma once
#include <deque>
#include <mutex>

namespace reef {

template <typename T>
class ThreadSafeQueue {
public:
    explicit ThreadSafeQueue(size_t capacity = 10000) : cap_(capacity) {}
    bool push(const T& v) {
        std::lock_guard<std::mutex> g(m_);
        if (q_.size() >= cap_) return false;
        q_.push_back(v);
        return true;
    }
    bool empty() const {
        std::lock_guard<std::mutex> g(m_);
        return q_.empty();
    }
    size_t size() const {
        std::lock_guard<std::mutex> g(m_);
        return q_.size();
    }
    // front() on an empty queue returns a default-constructed T
    T front() const {
        std::lock_guard<std::mutex> g(m_);
        return q_.empty() ? T() : q_.front();
    }
    void pop() {
        std::lock_guard<std::mutex> g(m_);
        if (!q_.empty()) q_.pop_front();
    }

private:
    mutable std::mutex m_;
    std::deque<T> q_;
    size_t cap_;
};

}  // namespace reef
