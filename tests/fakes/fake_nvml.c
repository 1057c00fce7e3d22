/* A stand-in for libnvidia-ml.so.1 for tests on a machine without a GPU: two GPUs, the first with 18 NVLink
 * links to a switch, the second with one link down. Only the read-only entry points the library uses. */
#include <string.h>

typedef int nvmlReturn_t;                 /* 0 = NVML_SUCCESS, 2 = invalid argument */
typedef struct { int index; } *nvmlDevice_t;

static struct { int index; } g_dev[2] = {{0}, {1}};
static int g_inits = 0;

nvmlReturn_t nvmlInit_v2(void) { g_inits++; return 0; }
nvmlReturn_t nvmlShutdown(void) { g_inits--; return 0; }
nvmlReturn_t nvmlDeviceGetCount_v2(unsigned int* n) { *n = 2; return 0; }
nvmlReturn_t nvmlDeviceGetHandleByIndex_v2(unsigned int i, nvmlDevice_t* d) { if (i > 1) return 2; *d = (nvmlDevice_t)&g_dev[i]; return 0; }
nvmlReturn_t nvmlDeviceGetHandleByPciBusId_v2(const char* pci, nvmlDevice_t* d) {
    if (!strcmp(pci, "0000:1B:00.0")) { *d = (nvmlDevice_t)&g_dev[0]; return 0; }
    if (!strcmp(pci, "0000:43:00.0")) { *d = (nvmlDevice_t)&g_dev[1]; return 0; }
    return 2;
}
nvmlReturn_t nvmlDeviceGetName(nvmlDevice_t d, char* name, unsigned int len) { strncpy(name, d->index ? "Fake B200 #1" : "Fake B200 #0", len); return 0; }
nvmlReturn_t nvmlDeviceGetNvLinkState(nvmlDevice_t d, unsigned int link, int* active) {
    if (link >= 18) return 2;
    *active = !(d->index == 1 && link == 7);
    return 0;
}
nvmlReturn_t nvmlDeviceGetNvLinkVersion(nvmlDevice_t d, unsigned int link, unsigned int* v) { (void)d; if (link >= 18) return 2; *v = 7; return 0; }
nvmlReturn_t nvmlDeviceGetNvLinkRemoteDeviceType(nvmlDevice_t d, unsigned int link, int* type) { (void)d; if (link >= 18) return 2; *type = 2; /* switch */ return 0; }
