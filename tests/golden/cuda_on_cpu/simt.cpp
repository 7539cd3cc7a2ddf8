// Blocks and threads of a CUDA launch on host threads (see cuda_runtime.h of this folder).
//
// One block runs at a time.  Its threads are host threads from a pool; they meet at
// __syncthreads() (threads that have returned from the kernel no longer count), and the lanes of
// a warp that a shuffle's mask names exchange their registers through a buffer of the warp.
#include "cuda_runtime.h"

#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

thread_local uint3 threadIdx;
thread_local uint3 blockIdx;
thread_local dim3 blockDim;
thread_local dim3 gridDim;

namespace {

struct Meeting {                       // a reusable barrier for a known number of threads
    int waiting = 0;
    unsigned long generation = 0;
};

struct Warp {
    std::mutex m;
    std::condition_variable cv;
    std::map<unsigned, Meeting> meetings;          // by mask: disjoint halves of a warp meet apart
    unsigned long long regs[32][6];
};

struct Block {
    std::mutex m;
    std::condition_variable cv;
    int live = 0;                      // threads that have not returned yet
    Meeting all;
    std::vector<Warp> warps;
};

Block* g_block = nullptr;
thread_local int t_linear = 0;         // the thread's number in its block

// The lanes of a warp that `mask` names wait for one another.
void meet(Warp& w, unsigned mask) {
    const int expected = __builtin_popcount(mask);
    std::unique_lock<std::mutex> lock(w.m);
    Meeting& mt = w.meetings[mask];                // looked up under the lock: lanes race to create it
    std::condition_variable& cv = w.cv;
    const unsigned long gen = mt.generation;
    if (++mt.waiting >= expected) {
        mt.waiting = 0;
        ++mt.generation;
        cv.notify_all();
    } else {
        cv.wait(lock, [&] { return mt.generation != gen; });
    }
}

// ---- a pool of host threads ------------------------------------------------------------------
struct Pool {
    std::mutex m;
    std::condition_variable work_cv, done_cv;
    std::vector<std::thread> threads;
    const std::function<void()>* body = nullptr;
    unsigned long job = 0;
    int wanted = 0, finished = 0;
    uint3 block_idx{};
    dim3 block_dim, grid_dim;

    void worker(int id) {
        unsigned long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(m);
                work_cv.wait(lock, [&] { return job != seen; });
                seen = job;
                if (id >= wanted) continue;
            }
            t_linear = id;
            blockDim = block_dim;
            gridDim = grid_dim;
            blockIdx = block_idx;
            threadIdx.x = id % block_dim.x;
            threadIdx.y = (id / block_dim.x) % block_dim.y;
            threadIdx.z = id / (block_dim.x * block_dim.y);
            (*body)();
            {   // a thread that has returned no longer takes part in the block's barriers
                std::unique_lock<std::mutex> lock(g_block->m);
                --g_block->live;
                if (g_block->live > 0 && g_block->all.waiting >= g_block->live) {
                    g_block->all.waiting = 0;
                    ++g_block->all.generation;
                    g_block->cv.notify_all();
                }
            }
            std::unique_lock<std::mutex> lock(m);
            if (++finished == wanted) done_cv.notify_all();
        }
    }

    void run_block(int nthreads, const std::function<void()>& fn) {
        while ((int)threads.size() < nthreads) {
            const int id = (int)threads.size();
            threads.emplace_back([this, id] { worker(id); });
            threads.back().detach();
        }
        std::unique_lock<std::mutex> lock(m);
        body = &fn;
        wanted = nthreads;
        finished = 0;
        ++job;
        work_cv.notify_all();
        done_cv.wait(lock, [&] { return finished == wanted; });
    }
};

Pool& pool() {
    static Pool* p = new Pool();       // never destroyed: its threads are detached
    return *p;
}

}  // namespace

void cpu_launch(dim3 grid, dim3 block, const std::function<void()>& thread_body) {
    const int nthreads = (int)(block.x * block.y * block.z);
    if (nthreads <= 0 || nthreads > 1024) {
        fprintf(stderr, "cpu_launch: a block of %d threads\n", nthreads);
        exit(2);
    }
    Pool& p = pool();
    for (unsigned bz = 0; bz < grid.z; ++bz)
        for (unsigned by = 0; by < grid.y; ++by)
            for (unsigned bx = 0; bx < grid.x; ++bx) {
                Block blk;
                blk.live = nthreads;
                blk.warps = std::vector<Warp>((nthreads + 31) / 32);
                g_block = &blk;
                p.block_idx = uint3{bx, by, bz};
                p.block_dim = block;
                p.grid_dim = grid;
                p.run_block(nthreads, thread_body);
                g_block = nullptr;
            }
}

void __syncthreads() {
    Block& b = *g_block;
    std::unique_lock<std::mutex> lock(b.m);
    const unsigned long gen = b.all.generation;
    if (++b.all.waiting >= b.live) {
        b.all.waiting = 0;
        ++b.all.generation;
        b.cv.notify_all();
    } else {
        b.cv.wait(lock, [&] { return b.all.generation != gen; });
    }
}

int cpu_lane_id() { return t_linear & 31; }

unsigned long long cpu_shfl(unsigned mask, unsigned long long bits, int src_lane) {
    Warp& w = g_block->warps[t_linear >> 5];
    const int lane = t_linear & 31;
    if (!((mask >> lane) & 1u)) {
        fprintf(stderr, "shuffle: lane %d is not in its own mask %08x\n", lane, mask);
        exit(2);
    }
    w.regs[lane][0] = bits;
    meet(w, mask);
    const unsigned long long got = w.regs[src_lane & 31][0];
    meet(w, mask);
    return got;
}

namespace {
float bf16_lo(uint32_t v) { uint32_t u = v << 16; float f; std::memcpy(&f, &u, 4); return f; }
float bf16_hi(uint32_t v) { uint32_t u = v & 0xffff0000u; float f; std::memcpy(&f, &u, 4); return f; }
}  // namespace

// Fragment layout of mma.sync.aligned.m16n8k16.row.col (g = lane / 4, t = lane % 4):
//   a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1], a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9]
//   b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g]
//   c0 = C[g][2t], c1 = C[g][2t+1], c2 = C[g+8][2t], c3 = C[g+8][2t+1]
void cpu_mma_m16n8k16_bf16(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                           float& c0, float& c1, float& c2, float& c3) {
    Warp& w = g_block->warps[t_linear >> 5];
    const int lane = t_linear & 31;
    w.regs[lane][0] = a0; w.regs[lane][1] = a1; w.regs[lane][2] = a2; w.regs[lane][3] = a3;
    w.regs[lane][4] = b0; w.regs[lane][5] = b1;
    meet(w, 0xffffffffu);
    auto a_at = [&](int row, int k) {
        const int src = (row & 7) * 4 + (k & 7) / 2;
        const uint32_t r = (uint32_t)w.regs[src][(row >> 3) + 2 * (k >> 3)];
        return (k & 1) ? bf16_hi(r) : bf16_lo(r);
    };
    auto b_at = [&](int k, int col) {
        const int src = col * 4 + (k & 7) / 2;
        const uint32_t r = (uint32_t)w.regs[src][4 + (k >> 3)];
        return (k & 1) ? bf16_hi(r) : bf16_lo(r);
    };
    const int g = lane >> 2, t = lane & 3;
    float* out[4] = {&c0, &c1, &c2, &c3};
    float add[4];
    for (int i = 0; i < 4; ++i) {
        const int row = g + 8 * (i >> 1), col = 2 * t + (i & 1);
        float s = 0.0f;
        for (int k = 0; k < 16; ++k) s += a_at(row, k) * b_at(k, col);
        add[i] = s;
    }
    meet(w, 0xffffffffu);
    for (int i = 0; i < 4; ++i) *out[i] += add[i];
}
