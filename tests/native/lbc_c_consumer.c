/* Plain C99 consumer of the C ABI: reads the header and one layer's index entry of an LBC
 * file through the shared library and prints what a host would pass to
 * lumen_moe_layer_prepare. Built and run by tests/test_abi.py (no GPU involved). */
#include <stdio.h>
#include <stdlib.h>

#include "lumen_moe.h"

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 3;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    unsigned char* data = (unsigned char*)malloc((size_t)n);
    if (!data || fread(data, 1, (size_t)n, f) != (size_t)n) return 4;
    fclose(f);
    lumen_lbc_header h;
    if (lumen_lbc_read_header(data, (size_t)n, &h) != LUMEN_MOE_OK) {
        printf("error %s\n", lumen_moe_last_error());
        return 5;
    }
    uint64_t gate[256], up[256], down[256];
    lumen_lbc_moe_layer L;
    if (lumen_lbc_read_moe_layer(data, (size_t)n, (uint32_t)atoi(argv[2]), &L, gate, up, down, 256) != LUMEN_MOE_OK) {
        printf("error %s\n", lumen_moe_last_error());
        return 6;
    }
    printf("version %u layers %u hidden %u experts %u top_k %u\n", h.version, h.num_layers, h.hidden_dim, h.num_experts,
           h.num_active_experts);
    printf("is_moe %u num_experts %u quant %d router_off %llu\n", L.is_moe, L.num_experts,
           (int)lumen_lbc_quant_to_moe(L.expert_gate_quant), (unsigned long long)L.router_weight.offset);
    if (L.is_moe)
        printf("expert0 %llu %llu %llu last_down %llu\n", (unsigned long long)gate[0], (unsigned long long)up[0],
               (unsigned long long)down[0], (unsigned long long)down[L.num_experts - 1]);
    free(data);
    return 0;
}
