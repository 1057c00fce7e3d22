/**
 * The switch (multimem) all-reduce kernel on ONE GPU, for profiling.
 *
 * A profiler that attaches to one process on one GPU cannot look at a kernel
 * that needs a peer. This helper builds a world of one rank whose memory is
 * bound to a multicast object with a single member, so that the zero-copy
 * switch variant runs its real instruction stream (multimem.ld_reduce,
 * multimem.st, the barriers) with the reduction over one contribution: the
 * output must equal the input. Whether a one-member multicast object can be
 * created depends on the driver and the fabric; when it cannot, the function
 * says so with a return code of -10 or below and touches nothing else.
 */
#include "../kernels/kernels.hpp"
#include "../core/types.hpp"
#include "driver_api.hpp"
#include <cstdio>
#include <cstring>

using namespace dccl;

extern "C" {

/**
 * All-reduce of `count` elements among one rank through the multicast mapping, `iters` calls.
 * host_in / host_out: `count` elements each. Returns 0, -10 (no multicast support), -11 (setting
 * up the memory failed; the reason goes to stderr), another negative value on a CUDA error, or
 * 100 + device status code when the kernel reported a failure.
 */
int dccl_emu_switch_single(int dtype, int op, size_t count, int ctas, int iters, const void* host_in, void* host_out) {
    const ncclDataType_t dt = (ncclDataType_t)dtype;
    const size_t es = size_of_type(dt);
    if (!es || !count || ctas < 1 || ctas > kMaxCtas || !nvls_supports(dt, (ncclRedOp_t)op)) return -2;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return -3;
    std::string err;
    const DriverApi* d = driver_api(&err);
    if (!d || !d->vmm_ok || !d->multicast_ok) return -10;
    CUdevice cu;
    int has_mc = 0;
    if (d->DeviceGet(&cu, dev) != CUDA_SUCCESS) return -3;
    d->DeviceGetAttribute(&has_mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu);
    if (!has_mc) return -10;

    const size_t bytes = (count * es + 255) / 256 * 256;
    const size_t stage = 2u << 20;
    const size_t user_off = kStageOff + 2 * stage;
    size_t total = user_off + 2 * bytes;

    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = 1;
    mp.size = total;
    size_t gran = 2u << 20, mg = 0;
    d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (d->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    total = (total + gran - 1) / gran * gran;
    mp.size = total;

    CUmemGenericAllocationHandle mem = 0, mc = 0;
    CUdeviceptr va = 0, mva = 0;
    bool mapped = false, mmapped = false, bound = false;
    uint32_t* status = nullptr;
    int rc = 0;
    CUresult r;
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    const char* step = "";
#define STEP(name, call) if (rc == 0 && (r = (call)) != CUDA_SUCCESS) { step = name; rc = -11; }
    STEP("cuMemCreate", d->MemCreate(&mem, total, &prop, 0));
    STEP("reserve", d->MemAddressReserve(&va, total, gran, 0, 0));
    STEP("map", d->MemMap(va, total, 0, mem, 0));
    if (rc == 0) mapped = true;
    STEP("set access", d->MemSetAccess(va, total, &acc, 1));
    STEP("cuMulticastCreate", d->MulticastCreate(&mc, &mp));
    STEP("cuMulticastAddDevice", d->MulticastAddDevice(mc, cu));
    STEP("cuMulticastBindMem", d->MulticastBindMem(mc, 0, mem, 0, total, 0));
    if (rc == 0) bound = true;
    STEP("reserve multicast", d->MemAddressReserve(&mva, total, gran, 0, 0));
    STEP("map multicast", d->MemMap(mva, total, 0, mc, 0));
    if (rc == 0) mmapped = true;
    STEP("set access multicast", d->MemSetAccess(mva, total, &acc, 1));
#undef STEP
    if (rc != 0) fprintf(stderr, "dccl one-rank switch run: %s failed: %s\n", step, cu_error(d, r).c_str());

    if (rc == 0 && (cudaMalloc((void**)&status, (ST_WORDS + 8) * sizeof(uint32_t)) != cudaSuccess ||
                    cudaMemset(status, 0, (ST_WORDS + 8) * sizeof(uint32_t)) != cudaSuccess ||
                    cudaMemset((void*)va, 0, kStageOff) != cudaSuccess)) rc = -4;
    if (rc == 0) {
        char* base = (char*)va;
        char* mbase = (char*)mva;
        cudaMemcpy(base + user_off, host_in, count * es, cudaMemcpyHostToDevice);
        cudaMemset(base + user_off + bytes, 0xEE, bytes);
        CollArgs a;
        memset(&a, 0, sizeof(a));
        a.comm.rank = 0;
        a.comm.nranks = 1;
        a.comm.pool[0] = base;
        a.comm.mc_pool = mbase;
        a.comm.status = status;
        a.comm.abort_word = status + ST_WORDS;
        a.comm.timeout_ns = 2000ull * 1000000ull;
        a.comm.stage_bytes = stage;
        a.io.send = base + user_off;
        a.io.recv = base + user_off + bytes;
        a.io.send_mc = mbase + user_off;
        a.io.recv_mc = mbase + user_off + bytes;
        a.symmetric = 1;
        a.mode = NV_ALLREDUCE;
        a.count = count;
        a.op = op;
        a.unroll = 8;
        LaunchCfg cfg;
        cfg.ctas = ctas;
        for (int it = 0; it < iters && rc == 0; it++) {
            a.seq = (uint32_t)(it + 1);
            a.parity = (int)(a.seq & 1u);
            if (launch_nvls(a, dt, cfg) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { rc = -5; break; }
            uint32_t st[ST_WORDS];
            cudaMemcpy(st, status, sizeof(st), cudaMemcpyDeviceToHost);
            if (st[ST_CODE] != DEV_OK) rc = 100 + (int)st[ST_CODE];
        }
        if (rc == 0) cudaMemcpy(host_out, base + user_off + bytes, count * es, cudaMemcpyDeviceToHost);
    }
    cudaDeviceSynchronize();
    cudaGetLastError();
    if (status) cudaFree(status);
    if (mmapped) d->MemUnmap(mva, total);
    if (mva) d->MemAddressFree(mva, total);
    if (bound) d->MulticastUnbind(mc, cu, 0, total);
    if (mc) d->MemRelease(mc);
    if (mapped) d->MemUnmap(va, total);
    if (va) d->MemAddressFree(va, total);
    if (mem) d->MemRelease(mem);
    return rc;
}

} // extern "C"
