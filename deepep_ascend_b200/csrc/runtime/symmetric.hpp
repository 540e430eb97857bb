// Symmetric memory for one NVLink domain: every rank allocates the same number of bytes, exports a handle,
// and maps every peer's allocation into its own address space, giving kernels a flat table of peer base
// pointers.  Two ways to build the table:
//   * processes, one per GPU: cudaIpc handles exchanged by the caller (torch.distributed all_gather_object);
//   * several virtual ranks inside one process on one GPU (protocol tests on a single GPU): plain pointers.
// Also owns the status block: pinned host memory mapped into the device, where kernels report failed waits
// and publish receive counts for the host.
// Optional CPU segment ("elastic" part of the buffer): `num_cpu_bytes` of host memory per rank that every rank's GPU
// can read, for tables that do not fit device memory (Engram storage).  It is a POSIX shared-memory object that
// the owner and every peer process map and pin with cudaHostRegister(mapped), so a kernel gets one device pointer
// per rank for it, exactly like the table of peer buffers.
// Parity: the role of csrc/kernels/backend/symmetric.hpp:14-319, csrc/utils/shared_memory.hpp:48-125 and the
// mapped host counters of csrc/elastic/buffer.hpp:127-142.
#pragma once
#include <cuda_runtime_api.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

#include "../kernels/api.h"
#include "coordinator.hpp"

namespace ep_host {

inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::ostringstream os;
        os << what << ": " << cudaGetErrorName(e) << " (" << cudaGetErrorString(e) << ")";
        throw BufferError(os.str());
    }
}

class SymmetricMemory {
public:
    SymmetricMemory(int rank, int num_ranks, int64_t num_bytes, int64_t num_cpu_bytes = 0)
        : rank_(rank), num_ranks_(num_ranks), bytes_(num_bytes), cpu_bytes_(num_cpu_bytes) {
        if (num_ranks < 1 || num_ranks > EP_MAX_RANKS || rank < 0 || rank >= num_ranks)
            throw BufferError("rank / num_ranks out of range");
        if (num_bytes < static_cast<int64_t>(EP_WORKSPACE_BYTES)) throw BufferError("buffer smaller than its workspace");
        cuda_check(cudaGetDevice(&device_), "cudaGetDevice");
        cuda_check(cudaMalloc(&local_, static_cast<size_t>(num_bytes)), "cudaMalloc(symmetric buffer)");
        cuda_check(cudaMemset(local_, 0, EP_WORKSPACE_BYTES), "cudaMemset(workspace)");
        void* host = nullptr;
        cuda_check(cudaHostAlloc(&host, EP_STATUS_WORDS * sizeof(uint64_t), cudaHostAllocMapped), "cudaHostAlloc(status block)");
        std::memset(host, 0, EP_STATUS_WORDS * sizeof(uint64_t));
        status_host_ = static_cast<uint64_t*>(host);
        cuda_check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_), host, 0), "cudaHostGetDevicePointer");
        for (int i = 0; i < EP_MAX_RANKS; ++i) peers_[i] = nullptr;
        peers_[rank_] = static_cast<uint8_t*>(local_);
        if (cpu_bytes_ > 0) {
            static std::atomic<uint64_t> serial{0};
            cpu_name_ = "/ep_b200_cpu_" + std::to_string(static_cast<long long>(getpid())) + "_" + std::to_string(serial.fetch_add(1));
            const int fd = shm_open(cpu_name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
            if (fd < 0) throw BufferError("shm_open(" + cpu_name_ + ") failed: " + std::strerror(errno));
            if (ftruncate(fd, static_cast<off_t>(cpu_bytes_)) != 0) {
                close(fd);
                shm_unlink(cpu_name_.c_str());
                throw BufferError("cannot size the CPU segment: " + std::string(std::strerror(errno)));
            }
            cpu_host_[rank_] = map_and_pin(fd, cpu_bytes_, &cpu_dev_[rank_]);
            close(fd);
        }
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }
    SymmetricMemory(const SymmetricMemory&) = delete;
    SymmetricMemory& operator=(const SymmetricMemory&) = delete;
    ~SymmetricMemory() { release(); }

    std::string export_handle() const {
        cudaIpcMemHandle_t h;
        cuda_check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
        return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
    }

    // handles[i] is rank i's export_handle(); maps every peer's buffer here
    void open_peers(const std::vector<std::string>& handles) {
        if (static_cast<int>(handles.size()) != num_ranks_) throw BufferError("one handle per rank is required");
        for (int i = 0; i < num_ranks_; ++i) {
            if (i == rank_) continue;
            if (handles[i].size() != sizeof(cudaIpcMemHandle_t)) throw BufferError("malformed IPC handle");
            cudaIpcMemHandle_t h;
            std::memcpy(&h, handles[i].data(), sizeof(h));
            void* p = nullptr;
            cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
            peers_[i] = static_cast<uint8_t*>(p);
            opened_[i] = true;
        }
        linked_ = true;
    }

    // all virtual ranks live in this process on this device
    static void link_local(const std::vector<SymmetricMemory*>& group) {
        for (auto* a : group) {
            if (static_cast<int>(group.size()) != a->num_ranks_) throw BufferError("group size != num_ranks");
            for (auto* b : group) {
                if (b->device_ != a->device_ || b->bytes_ != a->bytes_ || b->cpu_bytes_ != a->cpu_bytes_)
                    throw BufferError("virtual ranks must match");
                a->peers_[b->rank_] = static_cast<uint8_t*>(b->local_);
                a->cpu_dev_[b->rank_] = b->cpu_dev_[b->rank_];
            }
            a->linked_ = true;
        }
    }

    // ------------------------------------------------------------------ CPU segment
    int64_t cpu_bytes() const { return cpu_bytes_; }
    std::string export_cpu_name() const { return cpu_name_; }
    // names[i] is rank i's export_cpu_name(); maps and pins every peer's segment here.  Call unlink_cpu_name() on
    // every rank once all ranks are through (the mappings keep the memory alive).
    void open_cpu_peers(const std::vector<std::string>& names) {
        if (cpu_bytes_ == 0) return;
        if (static_cast<int>(names.size()) != num_ranks_) throw BufferError("one CPU segment name per rank is required");
        for (int i = 0; i < num_ranks_; ++i) {
            if (i == rank_) continue;
            const int fd = shm_open(names[i].c_str(), O_RDWR, 0600);
            if (fd < 0) throw BufferError("shm_open(" + names[i] + ") of a peer failed: " + std::strerror(errno));
            cpu_host_[i] = map_and_pin(fd, cpu_bytes_, &cpu_dev_[i]);
            close(fd);
        }
    }
    void unlink_cpu_name() {
        if (!cpu_name_.empty()) shm_unlink(cpu_name_.c_str());
        cpu_name_.clear();
    }
    // device-visible address of rank `r`'s CPU segment (null if absent or not mapped)
    uint8_t* cpu_segment(int r) const { return r >= 0 && r < num_ranks_ ? cpu_dev_[r] : nullptr; }
    uint8_t* cpu_segment_host() const { return static_cast<uint8_t*>(cpu_host_[rank_]); }

    RankCtx ctx(uint64_t timeout_ns) const {
        if (!linked_ && num_ranks_ > 1) throw BufferError("peers are not mapped yet");
        RankCtx c;
        c.rank = rank_;
        c.num_ranks = num_ranks_;
        for (int i = 0; i < EP_MAX_RANKS; ++i) c.peer_base[i] = peers_[i];
        c.status = status_dev_;
        c.timeout_ns = timeout_ns;
        return c;
    }

    bool release() {
        bool ok = true;
        for (int i = 0; i < EP_MAX_RANKS; ++i)
            if (opened_[i]) {
                ok = cudaIpcCloseMemHandle(peers_[i]) == cudaSuccess && ok;
                opened_[i] = false;
                peers_[i] = nullptr;
            }
        if (local_ != nullptr) {
            ok = cudaFree(local_) == cudaSuccess && ok;
            local_ = nullptr;
        }
        if (status_host_ != nullptr) {
            ok = cudaFreeHost(const_cast<uint64_t*>(status_host_)) == cudaSuccess && ok;
            status_host_ = nullptr;
        }
        for (int i = 0; i < EP_MAX_RANKS; ++i)
            if (cpu_host_[i] != nullptr) {
                ok = cudaHostUnregister(cpu_host_[i]) == cudaSuccess && ok;
                munmap(cpu_host_[i], static_cast<size_t>(cpu_bytes_));
                cpu_host_[i] = nullptr;
                cpu_dev_[i] = nullptr;
            }
        unlink_cpu_name();
        return ok;
    }

    int rank() const { return rank_; }
    int num_ranks() const { return num_ranks_; }
    int device() const { return device_; }
    int64_t bytes() const { return bytes_; }
    uint8_t* local() const { return static_cast<uint8_t*>(local_); }
    volatile uint64_t* status() const { return status_host_; }
    bool released() const { return local_ == nullptr; }

private:
    static void* map_and_pin(int fd, int64_t bytes, uint8_t** dev) {
        void* host = mmap(nullptr, static_cast<size_t>(bytes), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        if (host == MAP_FAILED) throw BufferError("mmap of a CPU segment failed: " + std::string(std::strerror(errno)));
        cudaError_t e = cudaHostRegister(host, static_cast<size_t>(bytes), cudaHostRegisterMapped | cudaHostRegisterPortable);
        if (e != cudaSuccess) {
            munmap(host, static_cast<size_t>(bytes));
            cuda_check(e, "cudaHostRegister(CPU segment)");
        }
        void* d = nullptr;
        cuda_check(cudaHostGetDevicePointer(&d, host, 0), "cudaHostGetDevicePointer(CPU segment)");
        *dev = static_cast<uint8_t*>(d);
        return host;
    }

    int rank_, num_ranks_, device_ = 0;
    int64_t bytes_;
    int64_t cpu_bytes_ = 0;
    std::string cpu_name_;
    void* cpu_host_[EP_MAX_RANKS] = {};
    uint8_t* cpu_dev_[EP_MAX_RANKS] = {};
    void* local_ = nullptr;
    uint8_t* peers_[EP_MAX_RANKS];
    bool opened_[EP_MAX_RANKS] = {};
    bool linked_ = false;
    volatile uint64_t* status_host_ = nullptr;
    uint64_t* status_dev_ = nullptr;
};

inline std::string describe_status(const volatile uint64_t* st) {
    static const char* kPhases[] = {"?", "grid barrier", "cross-GPU barrier", "dispatch count exchange", "dispatch load",
                                    "dispatch completion signal", "combine entry barrier", "combine load",
                                    "combine exit barrier", "low-latency receive count", "low-latency combine flag",
                                    "test flag", "pipeline credit", "tile flag", "GEMM pipeline", "dispatch row assignment of a CTA",
                                    "dispatch counts of a CTA"};
    std::ostringstream os;
    const uint64_t code = st[EP_STATUS_CODE], phase = st[EP_STATUS_PHASE];
    os << (code == EP_ERR_TIMEOUT ? "device wait timed out" : code == EP_ERR_BOUNDS ? "device bounds check failed"
                                                                                    : "device protocol error")
       << " on rank " << st[EP_STATUS_RANK] << " in phase '" << (phase < sizeof(kPhases) / sizeof(char*) ? kPhases[phase] : "?")
       << "' (peer " << static_cast<int64_t>(st[EP_STATUS_PEER]) << ", expected " << st[EP_STATUS_EXPECTED] << ", observed "
       << st[EP_STATUS_OBSERVED] << ")";
    return os.str();
}

}  // namespace ep_host
