// Exchange buffers between the GPUs of one node and the wait for the peers' announcements. The producers are the GEMV
// kernels themselves (decode.cuh: peers_put / peers_done); nothing here moves data.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;

// One thread per possible peer: spins (bounded) until that peer's epoch reaches the next one this rank waits for.
__global__ void __launch_bounds__(32) k_peer_wait(uint32_t * hdr, int rank_mask, uint64_t limit_ns) {
    const int r = threadIdx.x;
    const uint32_t want = hdr[XH_WAITED] + 1u;
    bool ok = true;
    if (r < 8 && (rank_mask >> r & 1)) {
        ok = false;
        uint64_t t0 = 0;
        for (uint32_t i = 0; i < (1u << 26); i++) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(hdr + r) : "memory");
            if ((int32_t) (seen - want) >= 0) { ok = true; break; }
            if ((i & 1023u) == 1023u) {
                uint64_t now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) { t0 = now; } else if (now - t0 > limit_ns) { break; }
            }
        }
    }
    if (!__all_sync(0xffffffffu, ok) && r == 0) { hdr[XH_EXPIRED] = 1u; }
    __syncwarp();
    if (r == 0) { hdr[XH_WAITED] = want; }
}

} // namespace

void peer_wait(uint32_t * local_header, int rank_mask, cudaStream_t st) {
    k_peer_wait<<<1, 32, 0, st>>>(local_header, rank_mask, dev::peer_wait_limit_ns());
    check_launch();
}

} // namespace b16
