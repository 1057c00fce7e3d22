/**
 * Driver of the ThreadSanitizer run of the kernel simulation (tests/test_kernel_sim.py): every emulated variant once
 * among four ranks, three calls each, plus a send/recv ring whose messages are longer than the FIFO and end in a
 * short chunk. Flags are host atomics with the release / acquire order the kernels ask for, so the sanitizer checks
 * that every data access between ranks is ordered by the protocol.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
extern "C" int dccl_emu_collective(const char*, const char*, int, int, int, size_t, int, int, int, size_t, int, size_t, const void*, void*);
extern "C" int dccl_emu_sendrecv_ring(int, size_t, int, int, int, const void*, void*);
int main(int argc, char** argv) {
    const char* kinds[] = {"allreduce", "reducescatter", "allgather", "broadcast", "reduce"};
    const char* algos[] = {"twoshot", "oneshot", "ring", "rabenseifner", "twoshot_ll"};
    int bad = 0;
    const int n = 4;
    for (const char* kind : kinds)
        for (const char* algo : algos) {
            if (strcmp(kind, "allreduce") && (!strcmp(algo, "rabenseifner"))) continue;
            if ((!strcmp(kind, "broadcast") || !strcmp(kind, "reduce")) && !strcmp(algo, "ring")) continue;
            if (!strcmp(algo, "twoshot_ll") && strcmp(kind, "allreduce") && strcmp(kind, "reduce")) continue;
            const size_t count = 4099;
            size_t in_e = !strcmp(kind, "reducescatter") ? count * n : count, out_e = !strcmp(kind, "allgather") ? count * n : count;
            std::vector<float> in(in_e * n), out(out_e * n);
            for (size_t i = 0; i < in.size(); i++) in[i] = (float)(i % 97) * 0.25f;
            int rc = dccl_emu_collective(kind, algo, n, 7, 0, count, 1, 2, 0, 0, 3, 1 << 20, in.data(), out.data());
            printf("%s %s rc=%d\n", kind, algo, rc);
            bad += rc != 0;
        }
    size_t nb = (5u << 20) + 4096;
    std::vector<unsigned char> in(n * nb), out(n * nb);
    for (size_t i = 0; i < in.size(); i++) in[i] = (unsigned char)(i * 7);
    int rc = dccl_emu_sendrecv_ring(n, nb, 1, 4, 2, in.data(), out.data());
    printf("sendrecv rc=%d\n", rc);
    return bad + (rc != 0);
}
