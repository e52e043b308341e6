// Several GPUs from the C++ host side (include/deep8/Deep8.h, "several GPUs"): a file-based rendezvous for the processes of
// one box, and the sum of replicated parameters' gradients over the ranks through peer-mapped GPU memory.  The GPU side is
// the C ABI's exchange entry points (include/d8k.h: d8k_peer_*, d8k_sum_shards); the order of calls is the one
// deep8_b200/dp.py's PeerAllReduce issues (copy-engine reduce-scatter, fixed-order sum, copy-engine all-gather).
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <thread>

#include <cuda_runtime.h>

#include "../../../include/deep8/Deep8.h"

namespace Deep8 {

namespace {

void d8kCheckDp(int rc) {
    if (rc == D8K_ERR_ARGUMENT) throw std::invalid_argument(d8k_last_error());
    if (rc != D8K_OK) throw std::runtime_error(d8k_last_error());
}

constexpr int kFlagWords = 64;  // per kind (ready, pulled, delivered): one word per writer, padded

}  // namespace

// ================================================================================================ FileRendezvous
FileRendezvous::FileRendezvous(std::string directory, int r, int w, double timeoutSeconds)
    : dir(std::move(directory)), myRank(r), worldSize(w), timeout(timeoutSeconds) {
    DEEP8_ARGUMENT_CHECK(w >= 1 && r >= 0 && r < w, "the rank must be in [0, world)");
}

void FileRendezvous::allGather(const void* mine, size_t bytes, void* all) {
    const long id = round++;
    auto path = [&](int r, bool tmp) { return dir + "/d8rv_" + std::to_string(id) + "_" + std::to_string(r) + (tmp ? ".tmp" : ".bin"); };
    {
        std::ofstream f(path(myRank, true), std::ios::binary | std::ios::trunc);
        if (!f) DEEP8_RUNTIME_ERROR("can not write into the rendezvous directory " << dir);
        f.write(static_cast<const char*>(mine), static_cast<std::streamsize>(bytes));
    }
    if (0 != std::rename(path(myRank, true).c_str(), path(myRank, false).c_str())) DEEP8_RUNTIME_ERROR("rename failed in " << dir);
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < worldSize; ++r) {
        char* dst = static_cast<char*>(all) + static_cast<size_t>(r) * bytes;
        if (r == myRank) {
            std::memcpy(dst, mine, bytes);
            continue;
        }
        for (;;) {
            std::ifstream f(path(r, false), std::ios::binary);
            if (f) {
                f.read(dst, static_cast<std::streamsize>(bytes));
                if (static_cast<size_t>(f.gcount()) == bytes) break;
            }
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout)
                DEEP8_RUNTIME_ERROR("rank " << r << " did not reach the rendezvous within " << timeout << " s");
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
        }
    }
}

void FileRendezvous::barrier() {
    std::vector<char> all(static_cast<size_t>(worldSize));
    char one = 1;
    allGather(&one, 1, all.data());
}

// ================================================================================================ PeerGradientSum
PeerGradientSum::PeerGradientSum(Executor* executor, Rendezvous* rendezvous, std::vector<Variable*> parameters, double timeoutMs)
    : rv(rendezvous), device(static_cast<GPUDevice*>(executor->getDevice())), params(std::move(parameters)), timeout(timeoutMs) {
    DEEP8_ARGUMENT_CHECK(nullptr != rv && !params.empty(), "PeerGradientSum needs a rendezvous and at least one parameter");
    world = rv->world();
    rank = rv->rank();
    DEEP8_ARGUMENT_CHECK(world <= 16, "at most 16 GPUs exchange through peer memory");
    for (auto p : params) {
        DEEP8_ARGUMENT_CHECK(p->updateGradient, "every parameter needs a gradient");
        DEEP8_ARGUMENT_CHECK(p->elementType() == params[0]->elementType(), "the parameters must share one element type");
        offsets.push_back(total);
        total += (p->gradient.size() + 127) / 128 * 128;  // every gradient starts on a 16-byte boundary for any element type
    }
    esize = params[0]->elementType().byteWidth;
    dtype = params[0]->elementType().id == DType::Float16 ? D8K_F16 : D8K_F32;
    DEEP8_ARGUMENT_CHECK(params[0]->elementType().id == DType::Float16 || params[0]->elementType().id == DType::Float32,
                         "type " << params[0]->elementType().name << " is not support");
    shardElems = ((total + world - 1) / world + 127) / 128 * 128;
    const size_t gradBytes = (total * esize + 255) / 256 * 256;
    stageBytes = (shardElems * esize + 255) / 256 * 256;
    offPartial = 0;
    offResult = gradBytes;
    offStage = 2 * gradBytes;
    offFlags = offStage + static_cast<size_t>(world) * stageBytes;
    const size_t bytes = offFlags + 3 * kFlagWords * 4;
    unsigned char handle[D8K_IPC_HANDLE_BYTES];
    void* ptr = nullptr;
    d8kCheckDp(d8k_peer_alloc(device->kernels, bytes, &ptr, handle));
    base = static_cast<char*>(ptr);
    peers.assign(static_cast<size_t>(world), nullptr);
    peers[rank] = base;
    if (world > 1) {
        std::vector<unsigned char> all(static_cast<size_t>(world) * D8K_IPC_HANDLE_BYTES);
        rv->allGather(handle, D8K_IPC_HANDLE_BYTES, all.data());
        for (int q = 0; q < world; ++q) {
            if (q == rank) continue;
            void* mapped = nullptr;
            d8kCheckDp(d8k_peer_open(device->kernels, all.data() + static_cast<size_t>(q) * D8K_IPC_HANDLE_BYTES, &mapped));
            peers[q] = static_cast<char*>(mapped);
        }
        rv->barrier();  // every rank has mapped every buffer before the first signal
    }
}

PeerGradientSum::~PeerGradientSum() {
    if (nullptr == base) return;
    device->synchronize();
    try {
        if (world > 1) rv->barrier();  // nobody unmaps or frees while a peer may still copy
        for (int q = 0; q < world; ++q)
            if (q != rank && peers[q]) d8k_peer_close(device->kernels, peers[q]);
        if (world > 1) rv->barrier();
    } catch (...) {
    }
    d8k_peer_free(device->kernels, base);
}

void* PeerGradientSum::flag(int owner, int kind, int writer) const {
    return peers[owner] + offFlags + (static_cast<size_t>(kind) * kFlagWords + writer) * 4;
}

void PeerGradientSum::sum() {
    d8k_ctx* c = device->kernels;
    auto copy = [&](void* dst, const void* src, size_t bytes) { d8kCheckDp(d8k_peer_copy(c, dst, src, bytes)); };
    if (1 == world) return;  // one rank: the gradients are the sums
    std::vector<int> order;
    for (int k = 1; k < world; ++k) order.push_back((rank + k) % world);  // at visit k every rank talks to a different peer
    auto flags = [&](int kind, bool mine) {
        std::vector<void*> f;
        for (int q : order) f.push_back(mine ? flag(rank, kind, q) : flag(q, kind, rank));
        return f;
    };
    if (!params.empty() && params[0]->executor) params[0]->executor->flush();
    if (step > 0) {  // the peers have pulled the previous partials before they are overwritten
        auto f = flags(1, true);
        d8kCheckDp(d8k_peer_wait(c, f.data(), static_cast<int>(f.size()), step, timeout));
    }
    ++step;
    for (size_t i = 0; i < params.size(); ++i)
        copy(base + offPartial + offsets[i] * esize, params[i]->gradient.raw(), params[i]->gradient.byteCount());
    {
        auto out = flags(0, false), in = flags(0, true);
        d8kCheckDp(d8k_peer_signal(c, out.data(), static_cast<int>(out.size()), step));  // my partial is ready
        d8kCheckDp(d8k_peer_wait(c, in.data(), static_cast<int>(in.size()), step, timeout));  // so are theirs
    }
    const size_t lo = std::min(static_cast<size_t>(rank) * shardElems, total), hi = std::min(lo + shardElems, total);
    const size_t n = hi - lo;
    if (n > 0)
        for (int q : order) copy(base + offStage + static_cast<size_t>(q) * stageBytes, peers[q] + offPartial + lo * esize, n * esize);
    {
        auto out = flags(1, false);
        d8kCheckDp(d8k_peer_signal(c, out.data(), static_cast<int>(out.size()), step));  // their partials may be rewritten
    }
    if (n > 0) {
        std::vector<const void*> srcs;
        for (int q = 0; q < world; ++q)
            srcs.push_back(q == rank ? base + offPartial + lo * esize : base + offStage + static_cast<size_t>(q) * stageBytes);
        d8kCheckDp(d8k_sum_shards(c, dtype, base + offResult + lo * esize, srcs.data(), world, n));
        for (int q : order) copy(peers[q] + offResult + lo * esize, base + offResult + lo * esize, n * esize);  // all-gather
    }
    {
        auto out = flags(2, false), in = flags(2, true);
        d8kCheckDp(d8k_peer_signal(c, out.data(), static_cast<int>(out.size()), step));  // my shard has been delivered
        d8kCheckDp(d8k_peer_wait(c, in.data(), static_cast<int>(in.size()), step, timeout));  // and so have theirs
    }
    for (size_t i = 0; i < params.size(); ++i)
        copy(params[i]->gradient.raw(), base + offResult + offsets[i] * esize, params[i]->gradient.byteCount());
}

void PeerGradientSum::synchronize() {
    int status = 0;
    d8kCheckDp(d8k_ctx_status(device->kernels, &status));
}

}  // namespace Deep8
