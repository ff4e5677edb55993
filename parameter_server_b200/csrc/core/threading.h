// Threading helpers: fixed thread pool with a final barrier, counting barrier,
// unbounded and byte-bounded blocking queues, and a one-producer prefetcher.
// Counterparts: util/threadpool.h:17-46, util/barrier.h:10-38,
// util/threadsafe_queue.h:8-48, util/threadsafe_limited_queue.h:10-72,
// util/producer_consumer.h:6-53.
#pragma once
#include <deque>
#include <queue>
#include "common.h"

namespace PS {

class ThreadPool {
 public:
  explicit ThreadPool(int num_workers) : num_workers_(std::max(1, num_workers)) {}
  ~ThreadPool() {
    if (!started_) return;
    { Lock l(mu_); waiting_to_finish_ = true; }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  typedef std::function<void()> Task;
  void add(const Task& task) { Lock l(mu_); tasks_.push_back(task); cv_.notify_one(); }
  void startWorkers() {
    started_ = true;
    for (int i = 0; i < num_workers_; ++i) threads_.emplace_back([this] { Run(); });
  }
 private:
  void Run() {
    while (true) {
      Task task;
      {
        ULock l(mu_);
        cv_.wait(l, [this] { return !tasks_.empty() || waiting_to_finish_; });
        if (tasks_.empty()) return;
        task = std::move(tasks_.front());
        tasks_.pop_front();
      }
      task();
    }
  }
  int num_workers_;
  std::deque<Task> tasks_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<std::thread> threads_;
  bool waiting_to_finish_ = false, started_ = false;
};

class Barrier {
 public:
  explicit Barrier(int num_threads) : num_to_block_(num_threads), num_to_exit_(num_threads) {}
  // true for exactly one of the threads of each round
  bool Block() {
    ULock l(mu_);
    if (--num_to_block_ == 0) cv_.notify_all();
    else cv_.wait(l, [this] { return num_to_block_ == 0; });
    return --num_to_exit_ == 0;
  }
 private:
  std::mutex mu_;
  std::condition_variable cv_;
  int num_to_block_, num_to_exit_;
};

template <typename T>
class ThreadsafeQueue {
 public:
  void push(T v) { { Lock l(mu_); q_.push(std::move(v)); } cv_.notify_one(); }
  void wait_and_pop(T& v) {
    ULock l(mu_);
    cv_.wait(l, [this] { return !q_.empty(); });
    v = std::move(q_.front());
    q_.pop();
  }
  bool try_pop(T& v) {
    Lock l(mu_);
    if (q_.empty()) return false;
    v = std::move(q_.front());
    q_.pop();
    return true;
  }
  size_t size() const { Lock l(mu_); return q_.size(); }
  bool empty() const { return size() == 0; }
 private:
  mutable std::mutex mu_;
  std::queue<T> q_;
  std::condition_variable cv_;
};

// Bounded by the total "capacity" units of the queued items; pop returns false
// once the producer has finished and the queue is drained.
template <typename T>
class ThreadsafeLimitedQueue {
 public:
  ThreadsafeLimitedQueue() {}
  explicit ThreadsafeLimitedQueue(size_t capacity) { setMaxCapacity(capacity); }
  void setMaxCapacity(size_t c) { max_capacity_ = c; }
  void push(const T& v, size_t capacity, bool finished = false) {
    PS_CHECK(!done_) << "push after the final element";
    if (capacity > max_capacity_) capacity = max_capacity_;
    ULock l(mu_);
    full_cv_.wait(l, [this, capacity] { return capacity + cur_capacity_ <= max_capacity_; });
    q_.push(std::make_pair(v, capacity));
    cur_capacity_ += capacity;
    done_ = finished;
    empty_cv_.notify_all();
  }
  bool pop(T& v) {
    ULock l(mu_);
    if (done_ && q_.empty()) return false;
    empty_cv_.wait(l, [this] { return !q_.empty(); });
    v = std::move(q_.front().first);
    cur_capacity_ -= q_.front().second;
    q_.pop();
    full_cv_.notify_all();
    return true;
  }
  size_t size() const { Lock l(mu_); return q_.size(); }
  bool empty() const { return size() == 0; }
 private:
  mutable std::mutex mu_;
  bool done_ = false;
  size_t max_capacity_ = 0, cur_capacity_ = 0;
  std::queue<std::pair<T, size_t>> q_;
  std::condition_variable empty_cv_, full_cv_;
};

// Runs `func(&item, &size)` on a background thread until it returns false and
// hands the items to the consumer through a byte-bounded queue.
template <class V>
class ProducerConsumer {
 public:
  ProducerConsumer() { setCapacity(1000); }
  explicit ProducerConsumer(int capacity_in_mb) { setCapacity(capacity_in_mb); }
  ~ProducerConsumer() { if (thr_.joinable()) thr_.join(); }
  void setCapacity(int mb) { queue_.setMaxCapacity((size_t)mb * 1024 * 1024); }
  void startProducer(const std::function<bool(V*, size_t*)>& func) {
    thr_ = std::thread([this, func] {
      V entry;
      bool done = false;
      while (!done) {
        size_t size = 0;
        done = !func(&entry, &size);
        queue_.push(entry, size, done);
      }
    });
  }
  bool pop(V* data) { return queue_.pop(*data); }
 private:
  ThreadsafeLimitedQueue<V> queue_;
  std::thread thr_;
};

}  // namespace PS
