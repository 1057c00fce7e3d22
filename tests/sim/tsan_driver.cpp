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
extern "C" void dccl_emu_set_peer_buffers(int);
extern "C" void dccl_emu_set_bcast_chunks(int);
extern "C" void dccl_emu_set_device_seq(int);
extern "C" void dccl_emu_set_switch_form(int);
extern "C" int dccl_emu_set_mix(const char*);
extern "C" int dccl_emu_all_to_all(int, size_t, int, int, const void*, void*);
extern "C" void dccl_emu_set_p2p_rendezvous(int);
extern "C" void dccl_emu_set_pipe(size_t, int);

static int run_one(const char* kind, const char* algo, int n, size_t count, int in_place, size_t misalign) {
    size_t in_e = !strcmp(kind, "reducescatter") ? count * n : count, out_e = !strcmp(kind, "allgather") ? count * n : count;
    std::vector<float> in(in_e * n), out(out_e * n);
    for (size_t i = 0; i < in.size(); i++) in[i] = (float)(i % 97) * 0.25f;
    int rc = dccl_emu_collective(kind, algo, n, 7, 0, count, n - 1, 2, in_place, misalign, 3, 8 << 20, in.data(), out.data());
    printf("%s %s n=%d count=%zu in_place=%d misalign=%zu rc=%d\n", kind, algo, n, count, in_place, misalign, rc);
    return rc != 0;
}
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
    // other world sizes, in place, unaligned; the zero-copy form on buffers every rank can address; the device-side counter
    for (int n2 : {2, 3, 8})
        for (const char* algo : algos) bad += run_one("allreduce", algo, n2, 1031, 0, 0);
    // worlds that are not a power of two: leader / follower pairs around the halving and doubling steps
    for (int n2 : {5, 6, 7}) bad += run_one("allreduce", "rabenseifner", n2, 40003, n2 == 6, n2 == 7 ? 4 : 0);
    bad += run_one("allreduce", "twoshot", 4, 5003, 1, 0);
    bad += run_one("allreduce", "ring", 4, 5003, 0, 4);
    bad += run_one("reducescatter", "twoshot", 4, 300000, 1, 0);      // large enough for the pushes and the fold to overlap in pieces
    dccl_emu_set_peer_buffers(1);
    bad += run_one("allreduce", "twoshot", 4, 40000, 0, 0);
    bad += run_one("allreduce", "twoshot", 8, 4099, 1, 0);
    bad += run_one("reducescatter", "twoshot", 4, 4096, 0, 0);
    // zero-copy broadcast (scatter and all-gather by peer loads, five chunks per shard) and reduce (root n - 1)
    dccl_emu_set_bcast_chunks(5);
    for (int n2 : {2, 3, 8}) {
        bad += run_one("broadcast", "twoshot", n2, 300000, 0, 0);
        bad += run_one("reduce", "twoshot", n2, 100003, n2 == 3, 0);
    }
    dccl_emu_set_bcast_chunks(0);
    dccl_emu_set_peer_buffers(0);
    dccl_emu_set_device_seq(1);
    for (const char* algo : algos) bad += run_one("allreduce", algo, 4, 1031, 0, 0);
    bad += run_one("broadcast", "oneshot", 4, 1031, 0, 0);
    bad += run_one("reduce", "oneshot", 4, 1031, 0, 0);
    dccl_emu_set_device_seq(0);
    // the switch kernels over the simulated multicast mapping: staged, pipelined all-reduce, pipelined broadcast / reduce
    for (int form = 0; form < 3; form++) {
        dccl_emu_set_switch_form(form);
        for (int n2 : {2, 4}) {
            if (form != 2) bad += run_one("allreduce", "nvls", n2, 40003, 0, 0);
            if (form == 0) { bad += run_one("reducescatter", "nvls", n2, 4099, 0, 0); bad += run_one("allgather", "nvls", n2, 4099, 0, 4); }
            if (form != 1) { bad += run_one("broadcast", "nvls", n2, 40003, 0, 4); bad += run_one("reduce", "nvls", n2, 40003, 1, 0); }
        }
    }
    dccl_emu_set_switch_form(0);
    dccl_emu_set_peer_buffers(1);       // zero-copy switch forms on multicast-mapped user buffers
    for (const char* kind : kinds) bad += run_one(kind, "nvls", 4, 40000, 0, 0);
    dccl_emu_set_peer_buffers(0);
    // sequences of different kernels in one world: rooted packet kernels between all-reduces, staged forms between packet forms
    for (const char* mix : {"allreduce:oneshot,broadcast:oneshot", "reduce:oneshot,allreduce:twoshot_ll", "broadcast:twoshot,reduce:twoshot_ll",
                            "allreduce:nvls,broadcast:nvls", "allreduce:ring,reducescatter:oneshot"}) {
        dccl_emu_set_mix(mix);
        for (const char* algo : {"oneshot", "twoshot_ll", "twoshot", "nvls"}) bad += run_one("allreduce", algo, 4, 1031, 0, 0);
    }
    dccl_emu_set_mix("");
    size_t nb = (5u << 20) + 4096;
    std::vector<unsigned char> in(n * nb), out(n * nb);
    for (size_t i = 0; i < in.size(); i++) in[i] = (unsigned char)(i * 7);
    int rc = dccl_emu_sendrecv_ring(n, nb, 1, 4, 2, in.data(), out.data());
    printf("sendrecv rc=%d\n", rc);
    {   // the all-to-all launch: receives and sends of every rank together, blocks longer than the FIFO
        const size_t blk = (4u << 20) + 4096;
        std::vector<unsigned char> ain(n * n * blk), aout(n * n * blk);
        for (size_t i = 0; i < ain.size(); i++) ain[i] = (unsigned char)(i * 13);
        const int arc = dccl_emu_all_to_all(n, blk, 2, 2, ain.data(), aout.data());
        printf("all_to_all rc=%d\n", arc);
        bad += arc != 0;
    }
    // large messages as rendezvous messages: stored straight into the receiver's buffer, through the FIFO after the
    // rendezvous, and both in one launch; then small messages again, which need the credit the direct messages returned
    for (int mode = 1; mode <= 3; mode++) {
        dccl_emu_set_p2p_rendezvous(mode);
        const size_t mb = (2u << 20) + 4096;
        std::vector<unsigned char> rin(n * 2 * mb), rout(n * 2 * mb);
        for (size_t i = 0; i < rin.size(); i++) rin[i] = (unsigned char)(i * 11);
        const int r1 = dccl_emu_sendrecv_ring(n, mb, 2, 3, 3, rin.data(), rout.data());
        const int r2 = dccl_emu_all_to_all(n, (1u << 20) + 64, 2, 2, rin.data(), rout.data());
        printf("rendezvous mode %d: sendrecv rc=%d all_to_all rc=%d\n", mode, r1, r2);
        bad += (r1 != 0) + (r2 != 0);
    }
    dccl_emu_set_p2p_rendezvous(0);
    // the pipelined switch forms with many small chunks and a switch group of its own size
    dccl_emu_set_switch_form(1);
    dccl_emu_set_pipe(4096, 2);
    bad += run_one("allreduce", "nvls", 4, 50001, 0, 0);
    bad += run_one("reducescatter", "nvls", 4, 20001, 0, 4);
    {   // a staging half of 64 KB under a 200 KB message: the chunk slots are reused as a ring, chunk numbers pass 24
        std::vector<float> rin(4 * 50001), rout(4 * 50001);
        for (size_t i = 0; i < rin.size(); i++) rin[i] = (float)(i % 89) * 0.5f;
        const int r1 = dccl_emu_collective("allreduce", "nvls", 4, 7, 0, 50001, 0, 7, 0, 0, 2, 64 << 10, rin.data(), rout.data());
        std::vector<float> sin(4 * 4 * 4099), sout(4 * 4099);
        for (size_t i = 0; i < sin.size(); i++) sin[i] = (float)(i % 83) * 0.5f;
        const int r2 = dccl_emu_collective("reducescatter", "nvls", 4, 7, 0, 4099, 0, 7, 0, 0, 2, 64 << 10, sin.data(), sout.data());
        printf("pipeline ring: allreduce rc=%d reducescatter rc=%d\n", r1, r2);
        bad += (r1 != 0) + (r2 != 0);
    }
    dccl_emu_set_pipe(16u << 20, 0);
    dccl_emu_set_switch_form(0);
    return bad + (rc != 0);
}
