/* The public header must be plain C and the library must load and answer without a GPU: dlopen, look up every
 * entry point named on the command line, call the ones that touch no device. */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "deepgemm_b200.h"

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (lib == NULL) {
        fprintf(stderr, "dlopen: %s\n", dlerror());
        return 3;
    }
    for (int i = 2; i < argc; ++i) {
        if (dlsym(lib, argv[i]) == NULL) {
            fprintf(stderr, "missing symbol %s\n", argv[i]);
            return 4;
        }
    }
    const char* (*version)(void) = (const char* (*)(void))dlsym(lib, "dg_version");
    int (*layout)(const dg_moe_config*, dg_moe_layout*) =
        (int (*)(const dg_moe_config*, dg_moe_layout*))dlsym(lib, "dg_mega_moe_buffer_layout");
    int (*alignment)(void) = (int (*)(void))dlsym(lib, "dg_get_token_alignment_for_mega_moe");
    const char* (*last_error)(void) = (const char* (*)(void))dlsym(lib, "dg_last_error");
    dg_moe_config cfg = {8, 256, 4096, 8, 7168, 2048, 0, 0};
    dg_moe_layout lay;
    memset(&lay, 0, sizeof(lay));
    if (layout(&cfg, &lay) != DG_OK) {
        fprintf(stderr, "layout: %s\n", last_error());
        return 5;
    }
    /* a bad configuration is refused with a message, not a crash */
    dg_moe_config bad = {3, 256, 4096, 8, 7168, 2048, 0, 0};
    dg_moe_layout unused;
    const int rc_bad = layout(&bad, &unused);
    printf("%s align=%d bytes=%lld pool_rows=%lld bad_rc=%d bad_msg=%s\n", version(), alignment(),
           (long long)lay.num_bytes, (long long)lay.pool_rows, rc_bad, rc_bad != DG_OK ? last_error() : "");
    dlclose(lib);
    return (lay.num_bytes > 0 && lay.pool_rows % 256 == 0 && rc_bad != DG_OK) ? 0 : 6;
}
