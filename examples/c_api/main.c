/* The flat C interface from plain C: a world of one rank, one all-reduce on host memory.
 * Build: cc main.c -I<prefix>/include -L<prefix>/lib -ldccl */
#include <dccl/dccl_c.h>
#include <stdio.h>

int main(void) {
    unsigned char id[128];
    void* comm = NULL;
    float in[4] = {1.f, 2.f, 3.f, 4.f}, out[4] = {0};
    if (dccl_get_unique_id(id) != 0 || dccl_comm_init_rank(&comm, 1, id, 0) != 0) return 1;
    if (dccl_all_reduce(in, out, 4, DCCL_FLOAT32, DCCL_SUM, comm, NULL) != 0) return 2;
    printf("rank %d of %d: %.0f %.0f %.0f %.0f (%s)\n", dccl_rank(comm), dccl_world_size(comm), out[0], out[1], out[2], out[3],
           dccl_error_string(0));
    return dccl_comm_finalize(comm);
}
