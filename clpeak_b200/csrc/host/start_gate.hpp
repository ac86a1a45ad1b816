// A reusable start barrier for the device threads of the multi-GPU driver.
//
// All parties call arrive(); the last one releases everybody so that the timed
// region of a test starts on every GPU at the same moment.  A party that never
// shows up (a thread that failed before the test) must not deadlock the others:
// arrive() gives up after `timeout` and marks the gate broken; from then on every
// arrive() returns immediately and the run carries on unsynchronised.
// leave() removes a party for good (a worker that stops early).
#pragma once

#include <chrono>
#include <condition_variable>
#include <mutex>

class StartGate {
public:
    explicit StartGate(int parties) : parties_(parties) {}

    // Returns true when all parties met, false when the gate is (or just became) broken.
    bool arrive(std::chrono::milliseconds timeout)
    {
        std::unique_lock<std::mutex> lk(m_);
        if (broken_ || parties_ <= 1)
            return !broken_;
        const unsigned long gen = generation_;
        if (++waiting_ >= parties_) {
            waiting_ = 0;
            ++generation_;
            cv_.notify_all();
            return true;
        }
        const bool met = cv_.wait_for(lk, timeout, [&] { return generation_ != gen || broken_; });
        if (!met) {
            broken_ = true;
            cv_.notify_all();
        }
        return !broken_;
    }

    void leave()
    {
        std::lock_guard<std::mutex> lk(m_);
        if (parties_ > 0)
            --parties_;
        if (parties_ > 0 && waiting_ >= parties_) {
            waiting_ = 0;
            ++generation_;
        }
        cv_.notify_all();
    }

    bool broken() const
    {
        std::lock_guard<std::mutex> lk(m_);
        return broken_;
    }

private:
    mutable std::mutex m_;
    std::condition_variable cv_;
    int parties_;
    int waiting_ = 0;
    unsigned long generation_ = 0;
    bool broken_ = false;
};
