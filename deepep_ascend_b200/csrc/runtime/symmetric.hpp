// Symmetric memory for one NVLink domain: every rank allocates the same number of bytes, exports a handle,
// and maps every peer's allocation into its own address space, giving kernels a flat table of peer base
// pointers.  Two ways to build the table:
//   * processes, one per GPU: cudaIpc handles exchanged by the caller (torch.distributed all_gather_object);
//   * several virtual ranks inside one process on one GPU (protocol tests on a single GPU): plain pointers.
// The local buffer is either a cudaMalloc allocation shared through cudaIpc handles, or (`use_vmm`) a CUDA virtual-memory
// allocation (cuMemCreate + cuMemMap) exported as a POSIX file descriptor that travels to the peers over a Unix-domain
// socket (SCM_RIGHTS) and is mapped there with cuMemImportFromShareableHandle: the scheme that also carries fabric handles
// across NVLink-connected nodes and that lets further allocations be mapped behind the same address range
// (csrc/kernels/backend/symmetric.hpp:22-87, csrc/utils/shared_memory.hpp:48-125 of the reference).
// Also owns the status block: pinned host memory mapped into the device, where kernels report failed waits
// and publish receive counts for the host.
// Optional CPU segment ("elastic" part of the buffer): `num_cpu_bytes` of host memory per rank that every rank's GPU
// can read, for tables that do not fit device memory (Engram storage).  It is a POSIX shared-memory object that
// the owner and every peer process map and pin with cudaHostRegister(mapped), so a kernel gets one device pointer
// per rank for it, exactly like the table of peer buffers.
// Parity: the role of csrc/kernels/backend/symmetric.hpp:14-319, csrc/utils/shared_memory.hpp:48-125 and the
// mapped host counters of csrc/elastic/buffer.hpp:127-142.
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <thread>
#include <type_traits>
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
// The driver's virtual-memory entry points, looked up at run time through the runtime API so that the extension does not
// link against libcuda (it must load on machines without a driver, e.g. for the CPU backend).
struct DriverApi {
    CUresult (*GetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*ExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*ImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*StreamWriteValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int) = nullptr;
    CUresult (*StreamWaitValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int) = nullptr;

    static const DriverApi& get() {
        static const DriverApi api = [] {
            DriverApi a;
            auto load = [](const char* name, auto& fn) {
                void* p = nullptr;
                cudaDriverEntryPointQueryResult q;
                if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
                    throw BufferError(std::string("the CUDA driver does not provide ") + name);
                fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(p);
            };
            load("cuMemGetAllocationGranularity", a.GetAllocationGranularity);
            load("cuMemCreate", a.Create);
            load("cuMemAddressReserve", a.AddressReserve);
            load("cuMemMap", a.Map);
            load("cuMemSetAccess", a.SetAccess);
            load("cuMemExportToShareableHandle", a.ExportToShareableHandle);
            load("cuMemImportFromShareableHandle", a.ImportFromShareableHandle);
            load("cuMemUnmap", a.Unmap);
            load("cuMemAddressFree", a.AddressFree);
            load("cuMemRelease", a.Release);
            load("cuStreamWriteValue64", a.StreamWriteValue64);
            load("cuStreamWaitValue64", a.StreamWaitValue64);
            return a;
        }();
        return api;
    }
};

inline void driver_check(CUresult r, const char* what) {
    if (r != CUDA_SUCCESS) throw BufferError(std::string(what) + " failed with CUDA driver error " + std::to_string(static_cast<int>(r)));
}

// One CUDA virtual-memory mapping: a physical allocation (own or imported) mapped read/write for `device`.
struct VmmMapping {
    CUmemGenericAllocationHandle handle = 0;
    CUdeviceptr ptr = 0;
    size_t size = 0;

    static CUmemAllocationProp props(int device) {
        CUmemAllocationProp p{};
        p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        p.location.id = device;
        p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        return p;
    }
    static size_t granularity(int device) {
        const CUmemAllocationProp p = props(device);
        size_t g = 0;
        driver_check(DriverApi::get().GetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
        return g;
    }
    void map(int device) {
        const size_t g = granularity(device);
        driver_check(DriverApi::get().AddressReserve(&ptr, size, g, 0, 0), "cuMemAddressReserve");
        driver_check(DriverApi::get().Map(ptr, size, 0, handle, 0), "cuMemMap");
        CUmemAccessDesc acc{};
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        driver_check(DriverApi::get().SetAccess(ptr, size, &acc, 1), "cuMemSetAccess");
    }
    void create(int device, size_t bytes) {
        const size_t g = granularity(device);
        size = (bytes + g - 1) / g * g;
        const CUmemAllocationProp p = props(device);
        driver_check(DriverApi::get().Create(&handle, size, &p, 0), "cuMemCreate");
        map(device);
    }
    int export_fd() const {
        int fd = -1;
        driver_check(DriverApi::get().ExportToShareableHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
        return fd;
    }
    void import_fd(int device, int fd, size_t bytes) {
        const size_t g = granularity(device);
        size = (bytes + g - 1) / g * g;
        driver_check(DriverApi::get().ImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                     "cuMemImportFromShareableHandle");
        map(device);
    }
    bool release() {
        bool ok = true;
        if (ptr != 0) {
            ok = DriverApi::get().Unmap(ptr, size) == CUDA_SUCCESS && ok;
            ok = DriverApi::get().AddressFree(ptr, size) == CUDA_SUCCESS && ok;
            ptr = 0;
        }
        if (handle != 0) {
            ok = DriverApi::get().Release(handle) == CUDA_SUCCESS && ok;
            handle = 0;
        }
        return ok;
    }
};

// Hands one file descriptor to `num_clients` peers over an abstract Unix-domain socket (SCM_RIGHTS), from a helper thread.
class FdServer {
public:
    FdServer(const std::string& name, int fd, int num_clients) : name_(name) {
        sock_ = socket(AF_UNIX, SOCK_STREAM, 0);
        if (sock_ < 0) throw BufferError("socket(AF_UNIX) failed");
        sockaddr_un addr{};
        addr.sun_family = AF_UNIX;
        std::memcpy(addr.sun_path + 1, name.data(), std::min(name.size(), sizeof(addr.sun_path) - 2));   // abstract: leading NUL
        const socklen_t len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + std::min(name.size(), sizeof(addr.sun_path) - 2));
        if (bind(sock_, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(sock_, num_clients + 1) != 0) {
            close(sock_);
            throw BufferError("cannot listen on the descriptor socket " + name + ": " + std::strerror(errno));
        }
        timeval tv{30, 0};   // a peer that never connects must not keep the thread forever
        setsockopt(sock_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        thread_ = std::thread([this, fd, num_clients] {
            for (int i = 0; i < num_clients; ++i) {
                const int c = accept(sock_, nullptr, nullptr);
                if (c < 0) break;
                send_fd(c, fd);
                close(c);
            }
        });
    }
    ~FdServer() { finish(); }
    void finish() {
        if (thread_.joinable()) thread_.join();
        if (sock_ >= 0) close(sock_);
        sock_ = -1;
    }
    static int fetch(const std::string& name) {
        sockaddr_un addr{};
        addr.sun_family = AF_UNIX;
        std::memcpy(addr.sun_path + 1, name.data(), std::min(name.size(), sizeof(addr.sun_path) - 2));
        const socklen_t len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + std::min(name.size(), sizeof(addr.sun_path) - 2));
        for (int attempt = 0; attempt < 200; ++attempt) {
            const int s = socket(AF_UNIX, SOCK_STREAM, 0);
            if (s < 0) break;
            if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) {
                const int fd = recv_fd(s);
                close(s);
                if (fd >= 0) return fd;
            } else {
                close(s);
            }
            std::this_thread::sleep_for(std::chrono::milliseconds(25));
        }
        throw BufferError("could not fetch the memory descriptor from " + name);
    }

private:
    static void send_fd(int sock, int fd) {
        char byte = 1, control[CMSG_SPACE(sizeof(int))] = {};
        iovec io{&byte, 1};
        msghdr msg{};
        msg.msg_iov = &io;
        msg.msg_iovlen = 1;
        msg.msg_control = control;
        msg.msg_controllen = sizeof(control);
        cmsghdr* c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int));
        std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
        sendmsg(sock, &msg, 0);
    }
    static int recv_fd(int sock) {
        char byte = 0, control[CMSG_SPACE(sizeof(int))] = {};
        iovec io{&byte, 1};
        msghdr msg{};
        msg.msg_iov = &io;
        msg.msg_iovlen = 1;
        msg.msg_control = control;
        msg.msg_controllen = sizeof(control);
        if (recvmsg(sock, &msg, 0) <= 0) return -1;
        cmsghdr* c = CMSG_FIRSTHDR(&msg);
        if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
        int fd = -1;
        std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
        return fd;
    }
    std::string name_;
    int sock_ = -1;
    std::thread thread_;
};

class SymmetricMemory {
public:
    SymmetricMemory(int rank, int num_ranks, int64_t num_bytes, int64_t num_cpu_bytes = 0, bool use_vmm = false)
        : rank_(rank), num_ranks_(num_ranks), bytes_(num_bytes), cpu_bytes_(num_cpu_bytes), use_vmm_(use_vmm) {
        if (num_ranks < 1 || num_ranks > EP_MAX_RANKS || rank < 0 || rank >= num_ranks)
            throw BufferError("rank / num_ranks out of range");
        if (num_bytes < static_cast<int64_t>(EP_WORKSPACE_BYTES)) throw BufferError("buffer smaller than its workspace");
        cuda_check(cudaGetDevice(&device_), "cudaGetDevice");
        if (use_vmm_) {
            cuda_check(cudaFree(nullptr), "CUDA context");   // the driver calls below need the primary context
            vmm_[rank_].create(device_, static_cast<size_t>(num_bytes));
            local_ = reinterpret_cast<void*>(vmm_[rank_].ptr);
        } else {
            cuda_check(cudaMalloc(&local_, static_cast<size_t>(num_bytes)), "cudaMalloc(symmetric buffer)");
        }
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

    bool uses_vmm() const { return use_vmm_; }

    // What the peers need to map this buffer: a cudaIpc handle, or (VMM) the name of a socket that hands out the file
    // descriptor of the allocation; the helper thread behind that socket serves every peer once.
    std::string export_handle() {
        if (use_vmm_) {
            static std::atomic<uint64_t> serial{0};
            const std::string name = "ep_b200_vmm_" + std::to_string(static_cast<long long>(getpid())) + "_" + std::to_string(serial.fetch_add(1));
            export_fd_ = vmm_[rank_].export_fd();
            fd_server_ = std::make_unique<FdServer>(name, export_fd_, num_ranks_ - 1);
            return "vmm:" + name;
        }
        cudaIpcMemHandle_t h;
        cuda_check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
        return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
    }

    // handles[i] is rank i's export_handle(); maps every peer's buffer here
    void open_peers(const std::vector<std::string>& handles) {
        if (static_cast<int>(handles.size()) != num_ranks_) throw BufferError("one handle per rank is required");
        if (use_vmm_) {
            for (int i = 0; i < num_ranks_; ++i) {
                if (i == rank_) continue;
                if (handles[i].rfind("vmm:", 0) != 0) throw BufferError("rank " + std::to_string(i) + " did not export a VMM allocation");
                const int fd = FdServer::fetch(handles[i].substr(4));
                vmm_[i].import_fd(device_, fd, static_cast<size_t>(bytes_));
                close(fd);
                peers_[i] = reinterpret_cast<uint8_t*>(vmm_[i].ptr);
            }
            linked_ = true;
            return;
        }
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

    // the socket thread has served every peer (call after all ranks are through open_peers)
    void finish_export() {
        if (fd_server_) fd_server_->finish();
        fd_server_.reset();
        if (export_fd_ >= 0) close(export_fd_);
        export_fd_ = -1;
    }

    bool release() {
        bool ok = true;
        finish_export();
        for (int i = 0; i < EP_MAX_RANKS; ++i)
            if (opened_[i]) {
                ok = cudaIpcCloseMemHandle(peers_[i]) == cudaSuccess && ok;
                opened_[i] = false;
                peers_[i] = nullptr;
            }
        if (use_vmm_) {
            for (int i = 0; i < EP_MAX_RANKS; ++i) ok = vmm_[i].release() && ok;
            local_ = nullptr;
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
    bool use_vmm_ = false;
    VmmMapping vmm_[EP_MAX_RANKS];
    std::unique_ptr<FdServer> fd_server_;
    int export_fd_ = -1;
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
