/* A plain C99 consumer of include/qlm_b200.h: proves the header is valid C (no C++ in the boundary) and that a
 * program linked against libqlm_b200.so gets status codes and messages, never an exit, without a GPU. */
#include <stdio.h>
#include <string.h>
#include "qlm_b200.h"

int main(void)
{
    qlmb_span sp;
    qlmb_moe_layer L;
    qlmb_ep_peers peers;
    int rc;
    memset(&sp, 0, sizeof sp); memset(&L, 0, sizeof L); memset(&peers, 0, sizeof peers);
    if (qlmb_version() < 1) { printf("version\n"); return 1; }
    rc = qlmb_encode(NULL, NULL, NULL, NULL, &sp, 1, 0, 128, 7, 1, NULL);
    if (rc != QLMB_E_ARG || !strstr(qlmb_last_error(), "qlmb_encode")) { printf("encode rc %d: %s\n", rc, qlmb_last_error()); return 2; }
    rc = qlmb_moe_forward(&L, NULL, NULL, NULL, NULL, NULL);
    if (rc == QLMB_OK) { printf("moe_forward accepted an empty layer\n"); return 3; }
    rc = qlmb_q4n_decode(NULL, NULL, NULL, 1024ull, 128, NULL);
    if (rc != QLMB_E_ARG) { printf("q4n rc %d\n", rc); return 4; }
    if (qlmb_comm_world(NULL) != 0 || qlmb_comm_rank(NULL) != -1) { printf("comm\n"); return 5; }
    printf("ok %d bytes per span, %d per layer descriptor\n", (int)sizeof(qlmb_span), (int)sizeof(qlmb_moe_layer));
    return 0;
}
