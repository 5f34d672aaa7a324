// LBC container: header and per-layer index reader for the MoE layer path.
//
// Host code only (no device work): reads the fixed header and the layer index table
// of an LBC file held in memory and hands out, per layer, what the MoE operator needs
// to prepare that layer from the layer blob as the backend uploads it -- the router
// slice, the per-expert gate/up/down byte offsets (relative to the layer blob), their
// quantisation tags, the FFN norm slice and the shared expert's slices.
//
// Format facts restated from the reference's reader and writer (little-endian):
//   header    crates/lumen-format/src/writer.rs:219-267, reader.rs:212-357
//   hyperparameters  writer.rs:270-331, reader.rs:383-481
//   tensor slice (24 bytes)  writer.rs:362-367, reader.rs:510-520
//   layer index entry  writer.rs:369-513, reader.rs:522-760
//   checksum  crates/lumen-format/src/crc.rs (CRC-32, reflected polynomial 0xEDB88320)
//   MoE metadata derived from an entry  crates/lumen-runtime/src/cuda/moe.rs:223-262
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/lumen_moe.h"

namespace lumen {
void set_last_error(const std::string& msg);
}

namespace {

constexpr uint32_t kMagic = 0x0143424Cu;  // "LBC\x01" (header.rs:7)
constexpr uint32_t kMaxVersion = 4;       // header.rs:9

struct Cursor {
    const uint8_t* p;
    size_t n, pos = 0;
    bool ok = true;
    bool need(size_t k) {
        if (!ok || k > n - pos) ok = false;
        return ok;
    }
    uint8_t u8() {
        if (!need(1)) return 0;
        return p[pos++];
    }
    uint32_t u32() {
        if (!need(4)) return 0;
        uint32_t v;
        memcpy(&v, p + pos, 4);
        pos += 4;
        return v;
    }
    uint64_t u64() {
        if (!need(8)) return 0;
        uint64_t v;
        memcpy(&v, p + pos, 8);
        pos += 8;
        return v;
    }
    float f32() {
        const uint32_t b = u32();
        float v;
        memcpy(&v, &b, 4);
        return v;
    }
    void skip(size_t k) {
        if (need(k)) pos += k;
    }
};

uint32_t crc32_update(uint32_t crc, const uint8_t* d, size_t n) {
    static uint32_t table[256];
    static bool built = false;
    if (!built) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int j = 0; j < 8; ++j) c = (c & 1u) ? (c >> 1) ^ 0xEDB88320u : c >> 1;
            table[i] = c;
        }
        built = true;
    }
    for (size_t i = 0; i < n; ++i) crc = (crc >> 8) ^ table[(crc ^ d[i]) & 0xFFu];
    return crc;
}

lumen_moe_status_t fail(lumen_moe_status_t st, const std::string& msg) {
    lumen::set_last_error(msg);
    return st;
}

// The scheme tags of quantization.rs:123-137; 0..12 are defined.
bool read_slice(Cursor& c, lumen_lbc_slice* s) {
    s->offset = c.u64();
    s->length = c.u64();
    s->quant = c.u8();
    s->present = 1;
    c.skip(7);
    return c.ok && s->quant <= 12;
}

bool slice_fits(const lumen_lbc_slice& s, uint64_t blob_len) {
    return s.offset + s.length >= s.offset && s.offset + s.length <= blob_len;
}

lumen_moe_status_t parse_header(Cursor& c, lumen_lbc_header* h) {
    memset(h, 0, sizeof(*h));
    const uint32_t magic = c.u32();
    if (!c.ok) return fail(LUMEN_MOE_INVALID_ARG, "LBC: unexpected end of data in the header");
    if (magic != kMagic) return fail(LUMEN_MOE_INVALID_ARG, "LBC: invalid magic");
    h->version = c.u32();
    if (c.ok && h->version > kMaxVersion) return fail(LUMEN_MOE_UNSUPPORTED, "LBC: unsupported version " + std::to_string(h->version));
    const uint8_t endian = c.u8();
    if (c.ok && endian > 1) return fail(LUMEN_MOE_INVALID_ARG, "LBC: invalid endianness byte");
    if (c.ok && endian == 1) return fail(LUMEN_MOE_UNSUPPORTED, "LBC: big-endian payloads are not supported");
    c.skip(3);
    const uint32_t stored_crc = c.u32();
    // hyperparameters
    const uint32_t hp_layers = c.u32();
    h->num_heads = c.u32();
    h->num_kv_heads = c.u32();
    h->head_dim = c.u32();
    h->hidden_dim = c.u32();
    h->intermediate_dim = c.u32();
    h->vocab_size = c.u32();
    h->max_seq_len = c.u32();
    c.skip(12);  // rope: present flag + 11 bytes either way
    h->num_experts = c.u32();
    h->num_active_experts = c.u32();
    h->norm_eps = c.f32();
    if (h->version >= 4) {
        if (c.u8() != 0) c.skip(16);  // GatedDeltaNet dimensions
    }
    // primary quantisation descriptor: scheme, group tag, group value, block bytes, scale flag, scale offset
    h->primary_quant = c.u8();
    c.skip(14);
    h->alignment = c.u64();
    h->num_layers = c.u32();
    h->has_expert_index = c.u8() != 0;
    c.skip(3);
    h->layer_index_offset = c.u64();
    c.skip(8);  // expert_index_offset
    h->payload_offset = c.u64();
    c.skip(48);  // embedding, final norm, output projection ranges
    if (h->version >= 2) c.skip(8);
    if (h->version >= 3) c.skip(24);
    if (!c.ok) return fail(LUMEN_MOE_INVALID_ARG, "LBC: unexpected end of data in the header");
    h->header_bytes = c.pos;
    // checksum over the header with its own field zeroed
    uint32_t crc = 0xFFFFFFFFu;
    const uint8_t zero[4] = {0, 0, 0, 0};
    crc = crc32_update(crc, c.p, 12);
    crc = crc32_update(crc, zero, 4);
    crc = crc32_update(crc, c.p + 16, c.pos - 16);
    crc ^= 0xFFFFFFFFu;
    if (crc != stored_crc) return fail(LUMEN_MOE_INVALID_ARG, "LBC: header checksum mismatch");
    if (h->alignment == 0 || (h->alignment & (h->alignment - 1)) != 0)
        return fail(LUMEN_MOE_INVALID_ARG, "LBC: alignment is not a power of two");
    if (h->num_layers != hp_layers) return fail(LUMEN_MOE_INVALID_ARG, "LBC: layer count mismatch between header and hyperparameters");
    return LUMEN_MOE_OK;
}

struct Entry {
    lumen_lbc_moe_layer info;
    std::vector<lumen_lbc_slice> gate, up, down;
};

// One layer index entry starting at the cursor. `keep` = false only advances.
lumen_moe_status_t parse_entry(Cursor& c, Entry* e, bool keep) {
    lumen_lbc_moe_layer& L = e->info;
    memset(&L, 0, sizeof(L));
    L.layer_offset_bytes = c.u64();
    L.layer_length_bytes = c.u64();
    lumen_lbc_slice s, dense[3];
    bool tags_ok = true;
    for (int i = 0; i < 4; ++i) tags_ok &= read_slice(c, &s);  // wq wk wv wo
    for (int i = 0; i < 3; ++i) tags_ok &= read_slice(c, &dense[i]);  // dense gate/up/down (zero length when MoE)
    tags_ok &= read_slice(c, &s);                                      // attn_norm
    tags_ok &= read_slice(c, &L.ffn_norm);
    // each optional section is there when at least 8 more bytes of data follow
    if (c.ok && c.pos + 8 <= c.n) {
        const uint8_t bias = c.u8();
        c.skip(7);
        for (int b = 0; b < 3; ++b)
            if (bias & (1u << b)) tags_ok &= read_slice(c, &s);
    }
    uint32_t ne = 0;
    if (c.ok && c.pos + 8 <= c.n) {
        ne = c.u32();
        const bool has_router = c.u8() != 0;
        c.skip(3);
        if (has_router) tags_ok &= read_slice(c, &L.router_weight);
        if (c.ok && (uint64_t)ne * 72 > c.n - c.pos) c.ok = false;
        if (c.ok) {
            if (keep) {
                e->gate.resize(ne);
                e->up.resize(ne);
                e->down.resize(ne);
            }
            lumen_lbc_slice g, u, d;
            for (uint32_t i = 0; i < ne && c.ok; ++i) {
                tags_ok &= read_slice(c, &g);
                tags_ok &= read_slice(c, &u);
                tags_ok &= read_slice(c, &d);
                if (keep) {
                    e->gate[i] = g;
                    e->up[i] = u;
                    e->down[i] = d;
                }
            }
        }
    }
    L.num_experts = ne;
    if (c.ok && c.pos + 8 <= c.n) {
        const uint32_t flags = c.u32();
        c.skip(4);
        for (int bit = 0; bit < 16 && c.ok; ++bit) {
            if (!(flags & (1u << bit))) continue;
            if (bit == 12) {  // layer type byte + padding
                L.layer_type = c.u8();
                L.has_layer_type = 1;
                c.skip(7);
                continue;
            }
            lumen_lbc_slice* dst = bit == 0 ? &L.shared_expert_gate : bit == 1 ? &L.shared_expert_up
                                 : bit == 2 ? &L.shared_expert_down : bit == 15 ? &L.ffn_gate_inp_shexp : &s;
            tags_ok &= read_slice(c, dst);
        }
    }
    if (!c.ok) return fail(LUMEN_MOE_INVALID_ARG, "LBC: unexpected end of data in the layer index");
    if (!tags_ok) return fail(LUMEN_MOE_UNSUPPORTED, "LBC: unknown quantisation scheme tag in the layer index");
    return LUMEN_MOE_OK;
}

}  // namespace

extern "C" {

lumen_moe_status_t lumen_lbc_read_header(const void* data, size_t bytes, lumen_lbc_header* out) {
    if (!data || !out) return fail(LUMEN_MOE_INVALID_ARG, "LBC: null argument");
    Cursor c{static_cast<const uint8_t*>(data), bytes};
    return parse_header(c, out);
}

lumen_moe_status_t lumen_lbc_read_moe_layer(const void* data, size_t bytes, uint32_t layer, lumen_lbc_moe_layer* out,
                                            uint64_t* gate_offs, uint64_t* up_offs, uint64_t* down_offs,
                                            uint32_t capacity) {
    if (!data || !out) return fail(LUMEN_MOE_INVALID_ARG, "LBC: null argument");
    Cursor c{static_cast<const uint8_t*>(data), bytes};
    lumen_lbc_header h;
    lumen_moe_status_t st = parse_header(c, &h);
    if (st != LUMEN_MOE_OK) return st;
    if (layer >= h.num_layers) return fail(LUMEN_MOE_INVALID_ARG, "LBC: layer index out of range");
    if (h.layer_index_offset > bytes) return fail(LUMEN_MOE_INVALID_ARG, "LBC: unexpected end of data in the layer index");
    c.pos = (size_t)h.layer_index_offset;
    Entry e;
    for (uint32_t l = 0; l <= layer; ++l) {
        st = parse_entry(c, &e, l == layer);
        if (st != LUMEN_MOE_OK) return st;
    }
    lumen_lbc_moe_layer& L = e.info;
    // every slice used by the operator lies inside the layer blob (index.rs:229-378)
    const uint64_t len = L.layer_length_bytes;
    bool fits = slice_fits(L.ffn_norm, len);
    if (L.router_weight.present) fits &= slice_fits(L.router_weight, len);
    for (const lumen_lbc_slice* s : {&L.shared_expert_gate, &L.shared_expert_up, &L.shared_expert_down, &L.ffn_gate_inp_shexp})
        if (s->present) fits &= slice_fits(*s, len);
    for (uint32_t i = 0; i < L.num_experts; ++i)
        fits &= slice_fits(e.gate[i], len) && slice_fits(e.up[i], len) && slice_fits(e.down[i], len);
    if (!fits) return fail(LUMEN_MOE_INVALID_ARG, "LBC: a tensor slice of layer " + std::to_string(layer) + " lies outside the layer blob");
    // a layer is MoE when it has a router and at least one expert (cuda/moe.rs:226-231)
    L.is_moe = (L.num_experts > 0 && L.router_weight.present) ? 1 : 0;
    if (L.is_moe) {
        L.expert_gate_quant = e.gate[0].quant;  // all experts share the scheme of expert 0 (cuda/moe.rs:245-247)
        L.expert_down_quant = e.down[0].quant;
        L.expert_gate_bytes = e.gate[0].length;
        L.expert_down_bytes = e.down[0].length;
        if (gate_offs || up_offs || down_offs) {
            if (!gate_offs || !up_offs || !down_offs) return fail(LUMEN_MOE_INVALID_ARG, "LBC: pass all three offset tables or none");
            if (capacity < L.num_experts) return fail(LUMEN_MOE_INVALID_ARG, "LBC: offset tables are smaller than the layer's expert count");
            for (uint32_t i = 0; i < L.num_experts; ++i) {
                gate_offs[i] = e.gate[i].offset;
                up_offs[i] = e.up[i].offset;
                down_offs[i] = e.down[i].offset;
            }
        }
    }
    *out = L;
    return LUMEN_MOE_OK;
}

int32_t lumen_lbc_quant_to_moe(uint32_t lbc_tag) {
    switch (lbc_tag) {  // quantization.rs:123-137
        case 3: return LUMEN_MOE_Q8_0;
        case 4: return LUMEN_MOE_Q4_0;
        case 2: return LUMEN_MOE_BF16;
        default: return -1;
    }
}

}  // extern "C"
