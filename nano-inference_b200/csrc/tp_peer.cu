// Peer-memory plumbing of tensor parallelism (one process per GPU): CUDA IPC handles of the
// model's exchange block, so that the decode kernel can store its tagged words straight into
// the other GPUs' copies over NVLink (the exchange inside the kernel needs nothing else), and
// a host-driven form of the same exchange for phase-by-phase launch sequences: after a sharded
// phase one small kernel stores the slice this GPU owns into every peer's copy of the
// exchanged vector, then tells each peer so through a flag in the peer's memory and waits -
// bounded - for the peers' flags.  The same sequence of exchanges runs on every GPU, so one
// monotonic epoch number per GPU identifies them.  The reference is single-GPU: no
// counterpart there.
//
// Why no later push can overwrite data a slower GPU still reads: the exchanges of a layer
// alternate (gate/up activations, down partial sums); a GPU pushes the next layer's
// activations only after it completed the down exchange in between, which needed the
// slower GPU's down push, which that GPU issued after its down phase had read the
// activations.  The same argument covers the partial sums (read in the next prologue, one
// exchange later) and the argmax candidates (one token later).
//
// Plain peer stores and loads only; every wait has a time budget,
// after which the kernel records MI_ERR_TIMEOUT and returns.
#include "model.cuh"

using namespace mi;

namespace {

constexpr int kMaxWorld = 8;

struct PeerXchg {
    uint8_t* local; uint8_t* peer[kMaxWorld];      // the exchanged buffer here and on every GPU (own slot unused)
    long long off[2], len[2];                      // up to two byte ranges this GPU owns
    int* flags_local; int* flags_peer[kMaxWorld];  // flags[src]: epoch of the last push that src completed into this GPU
    int* epoch;                                    // this GPU's count of completed exchanges
    int rank, world;
    int* err;
};

__global__ void __launch_bounds__(1024) tp_exchange_kernel(const PeerXchg X) {
    const int tid = threadIdx.x;
    const int epoch = *X.epoch + 1;
    for (int p = 0; p < X.world; p++) {
        if (p == X.rank) continue;
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            const long long off = X.off[r], len = X.len[r];
            if (len <= 0) continue;
            if (((off | len) & 15) == 0) {
                const uint4* s = reinterpret_cast<const uint4*>(X.local + off);
                uint4* d = reinterpret_cast<uint4*>(X.peer[p] + off);
                for (long long i = tid; i < (len >> 4); i += blockDim.x) d[i] = __ldcg(s + i);
            } else {                                   // every exchanged range is made of 8-byte words
                const unsigned long long* s = reinterpret_cast<const unsigned long long*>(X.local + off);
                unsigned long long* d = reinterpret_cast<unsigned long long*>(X.peer[p] + off);
                for (long long i = tid; i < (len >> 3); i += blockDim.x) d[i] = __ldcg(s + i);
            }
        }
    }
    __threadfence_system();                            // this thread's peer stores are performed before the flag below
    __syncthreads();
    __shared__ int s_ok;
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < X.world && tid != X.rank) {
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(X.flags_peer[tid] + X.rank), "r"(epoch) : "memory");
        const unsigned long long t0 = gtime_ns();
        int v;
        for (unsigned it = 0;; it++) {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(X.flags_local + tid) : "memory");
            if (v - epoch >= 0) break;
            if ((it & 63u) == 63u && gtime_ns() - t0 > kWaitBudgetNs) { s_ok = 0; break; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        *X.epoch = epoch;
        if (!s_ok) atomicMax(X.err, MI_ERR_TIMEOUT);
    }
}

}  // namespace

// Three handles of 64 bytes each: the exchange block (twice: the second slot is kept for layout compatibility) and the
// flag block of the host-driven exchange.
extern "C" int mi_tp_ipc_handles(mi_ctx* ctx, mi_model* m, void* out_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !out_host) return set_error(ctx, MI_ERR_INVALID, "tp_ipc_handles: null argument");
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    int st;
    if (!m->tp_flags) {
        // flag block: [kMaxWorld] flags, the epoch word, then the gathered argmax candidates [kMaxWorld] x {float, int}
        if ((st = dev_alloc(ctx, m, &m->tp_flags, 64))) return st;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t* h = reinterpret_cast<cudaIpcMemHandle_t*>(out_host);
    MI_CUDA(ctx, cudaIpcGetMemHandle(&h[0], m->P.xw));
    h[1] = h[0];
    MI_CUDA(ctx, cudaIpcGetMemHandle(&h[2], m->tp_flags));
    return MI_OK;
}

// all_host: [world][3] handles as gathered from every rank (own entry ignored).  After this call the model exchanges
// through peer memory (mi_tp_exchange) and its phase launches stop zeroing the exchanged buffers.
extern "C" int mi_tp_ipc_open(mi_ctx* ctx, mi_model* m, const void* all_host) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !all_host || !m->tp_flags) return set_error(ctx, MI_ERR_INVALID, "tp_ipc_open: call mi_tp_ipc_handles first");
    if (m->tp_world > kMaxWorld) return set_error(ctx, MI_ERR_LIMIT, "tp_ipc_open: at most %d GPUs", kMaxWorld);
    MI_CUDA(ctx, cudaSetDevice(ctx->device));
    const cudaIpcMemHandle_t* h = reinterpret_cast<const cudaIpcMemHandle_t*>(all_host);
    for (int r = 0; r < m->tp_world; r++) {
        for (int k = 0; k < 3; k += 2) {               // slot 1 repeats slot 0: one mapping serves both
            void* p = nullptr;
            if (r == m->tp_rank) p = k == 0 ? (void*)m->P.xw : (void*)m->tp_flags;
            else {
                MI_CUDA(ctx, cudaIpcOpenMemHandle(&p, h[r * 3 + k], cudaIpcMemLazyEnablePeerAccess));
                m->ipc_opened.push_back(p);
            }
            m->tp_peer[r][k] = p;
        }
        m->tp_peer[r][1] = m->tp_peer[r][0];
    }
    m->tp_peer_on = true;
    return MI_OK;
}

// Push this GPU's slice of one exchanged buffer (MI_TP_ACT, MI_TP_PART_DOWN of `layer`, MI_TP_BEST) to every peer and
// wait for theirs.  Asynchronous on the context's stream; every GPU must issue the same sequence of exchanges.
extern "C" int mi_tp_exchange(mi_ctx* ctx, mi_model* m, int which, int layer) {
    if (!ctx) return MI_ERR_INVALID;
    if (!m || !m->tp_peer_on) return set_error(ctx, MI_ERR_INVALID, "tp_exchange: peer memory is not set up (mi_tp_ipc_open)");
    PeerXchg X{};
    X.rank = m->tp_rank; X.world = m->tp_world; X.err = ctx->d_err;
    X.flags_local = m->tp_flags; X.epoch = m->tp_flags + kMaxWorld;
    for (int r = 0; r < m->tp_world; r++) X.flags_peer[r] = reinterpret_cast<int*>(m->tp_peer[r][2]);
    int g0, g1;
    if (which == MI_TP_ACT) {
        // tagged words of the q8_0 vector: 8 value words per block, then one scale word per block
        mi_tp_partition(m->FF / 32, m->tp_rank, m->tp_world, &g0, &g1);
        X.local = reinterpret_cast<uint8_t*>(m->P.xw);
        for (int r = 0; r < m->tp_world; r++) X.peer[r] = reinterpret_cast<uint8_t*>(m->tp_peer[r][0]);
        X.off[0] = ((long long)m->P.xo.act + (long long)g0 * 8) * 8; X.len[0] = (long long)(g1 - g0) * 64;
        X.off[1] = ((long long)m->P.xo.act + m->FF / 4 + g0) * 8; X.len[1] = (long long)(g1 - g0) * 8;
    } else if (which == MI_TP_PART_DOWN) {
        if (layer < 0 || layer >= m->L) return set_error(ctx, MI_ERR_INVALID, "tp_exchange: bad layer");
        mi_tp_partition((m->E + 31) / 32, m->tp_rank, m->tp_world, &g0, &g1);
        X.local = reinterpret_cast<uint8_t*>(m->P.xw);
        for (int r = 0; r < m->tp_world; r++) X.peer[r] = reinterpret_cast<uint8_t*>(m->tp_peer[r][0]);
        X.off[0] = ((long long)m->P.xo.down + (long long)g0 * 32) * 8; X.len[0] = (long long)(g1 - g0) * 256;
    } else if (which == MI_TP_BEST) {
        // candidates live behind the flags: [kMaxWorld + 8 ints] then [world] x {float, int}; this GPU's own entry first
        // moves from the model's {value, token} pair into its slot, then the slot goes to the peers
        int* gathered = m->tp_flags + 2 * kMaxWorld;
        MI_CUDA(ctx, cudaMemcpyAsync(gathered + 2 * m->tp_rank, m->best_buf, 8, cudaMemcpyDeviceToDevice, ctx->stream));
        X.local = reinterpret_cast<uint8_t*>(m->tp_flags);
        for (int r = 0; r < m->tp_world; r++) X.peer[r] = reinterpret_cast<uint8_t*>(m->tp_peer[r][2]);
        X.off[0] = (long long)(2 * kMaxWorld + 2 * m->tp_rank) * 4; X.len[0] = 8;
    } else {
        return set_error(ctx, MI_ERR_INVALID, "tp_exchange: region %d is not exchanged", which);
    }
    tp_exchange_kernel<<<1, 1024, 0, ctx->stream>>>(X);
    MI_CUDA(ctx, cudaGetLastError());
    if (which == MI_TP_BEST) return mi_tp_pick(ctx, m, m->tp_flags + 2 * kMaxWorld, m->tp_world);
    return MI_OK;
}
