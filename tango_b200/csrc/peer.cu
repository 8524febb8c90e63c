// Cross-GPU rendezvous for the GPUs of one node, over peer memory (plain NVLink stores and loads; no multicast).
//
// Every rank owns a slot array of 2 * world 64-bit words that all ranks have mapped.  In round e (e = 1, 2, ...) rank r
// stores (e << 32 | bits of its fp32 value) into word (e & 1) * world + r of EVERY rank's array with a system-scope
// release store, then waits until the `world` words of that round in its OWN array carry round e (system-scope
// acquire loads), and returns the maximum of the values.  One launch is therefore both a barrier -- everything the
// rank wrote to peer memory in earlier kernels of the stream is visible to a rank that has seen its word -- and an
// all-reduce(max) of one float.  Two banks of words (round parity) keep a fast rank's round e + 1 from overwriting a
// word that a slow rank has not read yet: a rank can only reach round e + 2 after every rank has written round
// e + 1, i.e. after every rank has finished reading round e.
//
// The wait is bounded (limit_ns of %globaltimer, two seconds by default): on expiry the kernel stores TANGO_ETIMEOUT
// in the status word and returns the maximum of the values it did see, so a missing peer can never hang the GPU.  The
// round counter still advances, and a late peer's word stays in its bank, so the ranks meet again in the next round.
#include <cstring>

#include "common.cuh"

namespace tango {

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(64) peer_sync_kernel(unsigned long long *const *slots, int rank, int world,
                                                       unsigned long long *round_word, const float *val_in,
                                                       float *val_out, int *status,
                                                       unsigned long long limit_ns) {
    __shared__ float vals[64];
    const int t = threadIdx.x;
    const unsigned long long e = *round_word + 1ull;          // every thread reads before thread 0 advances it
    __syncthreads();
    if (t == 0) *round_word = e;
    const float mine = val_in ? *val_in : 0.f;
    const int bank = (int)(e & 1ull) * world;
    float got = 0.f;
    if (t < world) {
        __threadfence_system();                                // earlier writes of this GPU before the flag
        st_release_sys(slots[t] + bank + rank, (e << 32) | (unsigned long long)__float_as_uint(mine));
        const unsigned long long *my_word = slots[rank] + bank + t;
        const unsigned long long t0 = global_timer_ns();
        unsigned long long v = ld_acquire_sys(my_word);
        while ((v >> 32) < e) {
            if (global_timer_ns() - t0 > limit_ns) {
                if (status) atomicExch(status, TANGO_ETIMEOUT);
                break;
            }
            __nanosleep(100);
            v = ld_acquire_sys(my_word);
        }
        // a word that still carries an older round holds an older value: it does not take part
        got = ((v >> 32) >= e) ? __uint_as_float((unsigned int)(v & 0xffffffffull)) : 0.f;
    }
    vals[t] = (t < world && (got == got)) ? got : 0.f;
    __syncthreads();
    if (t == 0 && val_out) {
        float m = vals[0];
        for (int k = 1; k < world; ++k) m = fmaxf(m, vals[k]);
        *val_out = m;
    }
}

}  // namespace tango

using namespace tango;

// ---- set-up helpers (host side, once per buffer): memory that other processes of the node can map.
// The buffer is a plain cudaMalloc allocation, so its address is the base address cudaIpcGetMemHandle wants, and a
// peer opens the handle with ITS OWN device current, which maps the memory for kernels of that device (with peer
// access enabled on demand).

extern "C" int tango_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle64) {
    if (bytes <= 0 || !ptr || !handle64) return TANGO_EINVAL;
    void *p = nullptr;
    TANGO_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        TANGO_CUDA_TRY(e);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    return TANGO_OK;
}

extern "C" int tango_peer_open(const unsigned char *handle64, void **ptr) {
    if (!handle64 || !ptr) return TANGO_EINVAL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *p = nullptr;
    TANGO_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return TANGO_OK;
}

extern "C" int tango_peer_close(void *ptr) {
    if (!ptr) return TANGO_OK;
    TANGO_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return TANGO_OK;
}

extern "C" int tango_peer_free(void *ptr) {
    if (!ptr) return TANGO_OK;
    TANGO_CUDA_TRY(cudaFree(ptr));
    return TANGO_OK;
}

extern "C" int tango_enable_peer_access(int peer_device) {
    int cur = -1;
    TANGO_CUDA_TRY(cudaGetDevice(&cur));
    if (peer_device == cur) return TANGO_OK;
    int can = 0;
    TANGO_CUDA_TRY(cudaDeviceCanAccessPeer(&can, cur, peer_device));
    if (!can) return TANGO_EINVAL;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();   // not an error: PyTorch or an earlier call enabled it
        return TANGO_OK;
    }
    TANGO_CUDA_TRY(e);
    return TANGO_OK;
}

extern "C" int tango_peer_sync(uint64_t *const *slots, int rank, int world, uint64_t *round_word, const float *val_in,
                               float *val_out, int *status, int64_t limit_ns, tango_stream_t stream) {
    if (!slots || !round_word || world < 1 || world > 64 || rank < 0 || rank >= world) return TANGO_EINVAL;
    const unsigned long long limit = limit_ns > 0 ? (unsigned long long)limit_ns : 2000000000ull;
    peer_sync_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(reinterpret_cast<unsigned long long *const *>(slots), rank, world,
                                                         reinterpret_cast<unsigned long long *>(round_word), val_in,
                                                         val_out, status, limit);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}
