// Host-side life cycle of one communication buffer.
//
//   Idle -> Active (an operation is being validated / launched) -> Idle
//        -> Poisoned (a device wait ran out, a launch failed, or an operation was abandoned half-way)
//        -> Destroying -> Destroyed
//
// Every accepted operation gets a strictly increasing generation number.  A poisoned buffer refuses new
// operations but can still be destroyed; destroy() may be retried and is idempotent.  Plain C++17 with no CUDA
// or torch dependency so that it is unit-tested on the host.
// Parity: the operation coordinator of the reference's NPU backend
// (csrc/backends/ascend/elastic/operation_coordinator.hpp:9-315).
#pragma once
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>

namespace ep_host {

class BufferError : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

enum class BufferState { Idle, Active, Poisoned, Destroying, Destroyed };

inline const char* to_string(BufferState s) {
    switch (s) {
        case BufferState::Idle: return "idle";
        case BufferState::Active: return "active";
        case BufferState::Poisoned: return "poisoned";
        case BufferState::Destroying: return "destroying";
        default: return "destroyed";
    }
}

class OperationCoordinator {
public:
    // Admit one operation; throws if the buffer cannot take it.
    uint64_t begin(const char* what) {
        std::lock_guard<std::mutex> lock(mu_);
        switch (state_) {
            case BufferState::Idle: break;
            case BufferState::Active:
                throw BufferError(std::string(what) + ": another operation is being launched on this buffer");
            case BufferState::Poisoned:
                throw BufferError(std::string(what) + ": buffer is poisoned (" + reason_ + "); destroy and recreate it");
            default:
                throw BufferError(std::string(what) + ": buffer is " + to_string(state_));
        }
        state_ = BufferState::Active;
        active_generation_ = ++generation_;
        return active_generation_;
    }

    // Finish the operation admitted with `generation`.  ok == false poisons the buffer.
    void complete(uint64_t generation, bool ok, const std::string& why = "") {
        std::lock_guard<std::mutex> lock(mu_);
        if (state_ != BufferState::Active || generation != active_generation_) {
            if (state_ == BufferState::Idle || state_ == BufferState::Active) poison_locked("completion of a stale operation");
            return;
        }
        if (ok) state_ = BufferState::Idle;
        else poison_locked(why.empty() ? "operation failed" : why);
    }

    void poison(const std::string& why) {
        std::lock_guard<std::mutex> lock(mu_);
        if (state_ == BufferState::Idle || state_ == BufferState::Active) poison_locked(why);
    }

    // Returns true when the caller must release the resources now (first successful entry).
    bool begin_destroy() {
        std::lock_guard<std::mutex> lock(mu_);
        if (state_ == BufferState::Destroyed || state_ == BufferState::Destroying) return false;
        state_ = BufferState::Destroying;
        return true;
    }
    // released == false leaves the buffer poisoned so destroy() can be retried.
    void end_destroy(bool released) {
        std::lock_guard<std::mutex> lock(mu_);
        if (state_ != BufferState::Destroying) return;
        if (released) state_ = BufferState::Destroyed;
        else {
            state_ = BufferState::Poisoned;
            if (reason_.empty()) reason_ = "destroy failed";
        }
    }

    BufferState state() const {
        std::lock_guard<std::mutex> lock(mu_);
        return state_;
    }
    uint64_t generation() const {
        std::lock_guard<std::mutex> lock(mu_);
        return generation_;
    }
    std::string reason() const {
        std::lock_guard<std::mutex> lock(mu_);
        return reason_;
    }
    bool usable() const { return state() == BufferState::Idle; }

private:
    void poison_locked(const std::string& why) {
        state_ = BufferState::Poisoned;
        if (reason_.empty()) reason_ = why;
    }
    mutable std::mutex mu_;
    BufferState state_ = BufferState::Idle;
    uint64_t generation_ = 0;
    uint64_t active_generation_ = 0;
    std::string reason_;
};

// RAII admission: an operation that unwinds without commit() poisons the buffer.
class OperationScope {
public:
    OperationScope(OperationCoordinator& c, const char* what) : c_(c), generation_(c.begin(what)) {}
    ~OperationScope() {
        if (!done_) c_.complete(generation_, false, "operation abandoned before launch completed");
    }
    void commit() {
        c_.complete(generation_, true);
        done_ = true;
    }
    uint64_t generation() const { return generation_; }

private:
    OperationCoordinator& c_;
    uint64_t generation_;
    bool done_ = false;
};

}  // namespace ep_host
