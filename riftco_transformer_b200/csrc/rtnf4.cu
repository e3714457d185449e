// Index of an RTNF4S1 packed-model-state stream (host code only).
//
// Restates the checks of the reference's parser, parse_packed_model_state
// (src/c_api/model_state.cpp:165-297), without copying any payload: the result
// is a table of byte offsets into the caller's buffer.
#include "b2_common.cuh"

#include <cstring>
#include <limits>

namespace b2 {
namespace {

struct Reader {
    const uint8_t* base;
    uint64_t size;
    uint64_t at;

    uint64_t remaining() const { return size - at; }
    // 0 on success; the cursor moves past `count` bytes
    int32_t take(uint64_t count, const char* what, uint64_t* offset) {
        if (count > remaining()) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "truncated packed model state: %s", what);
        }
        *offset = at;
        at += count;
        return B2_STATUS_OK;
    }
    int32_t u32(const char* what, uint32_t* value) {
        uint64_t off = 0;
        B2_TRY(take(4, what, &off));
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(base[off + i]) << (8 * i);
        *value = v;
        return B2_STATUS_OK;
    }
    int32_t u64(const char* what, uint64_t* value) {
        uint64_t off = 0;
        B2_TRY(take(8, what, &off));
        uint64_t v = 0;
        for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(base[off + i]) << (8 * i);
        *value = v;
        return B2_STATUS_OK;
    }
};

constexpr uint8_t kMagic[8] = {'R', 'T', 'N', 'F', '4', 'S', '1', '\0'};

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int32_t b2_rtnf4_index(const uint8_t* stream, uint64_t bytes, b2_rtnf4_entry* entries, uint64_t capacity,
                                  uint64_t* count_out) {
    clear_error();
    if (stream == nullptr || count_out == nullptr || (entries == nullptr && capacity != 0)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "packed model state index needs a stream and a count pointer");
    }
    Reader r{stream, bytes, 0};
    uint64_t off = 0;
    B2_TRY(r.take(sizeof(kMagic), "magic", &off));
    if (std::memcmp(stream + off, kMagic, sizeof(kMagic)) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "unknown packed model state format");
    }
    uint64_t count = 0;
    B2_TRY(r.u64("weight count", &count));
    constexpr uint64_t kMinimumEntryBytes = 80;
    if (count == 0 || count > r.remaining() / kMinimumEntryBytes) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "packed model state weight count is inconsistent with its size");
    }
    for (uint64_t index = 0; index < count; ++index) {
        b2_rtnf4_entry e;
        std::memset(&e, 0, sizeof(e));
        uint64_t rank = 0;
        B2_TRY(r.u64("rank", &rank));
        if (rank != 2) return fail(B2_STATUS_INVALID_ARGUMENT, "packed decoder Linear weights must have rank two");
        B2_TRY(r.u64("block size", &e.block_size));
        B2_TRY(r.u64("packed code count", &e.n_codes));
        B2_TRY(r.u64("block scale count", &e.n_fp32_scales));
        B2_TRY(r.u64("scale code count", &e.n_scale_codes));
        B2_TRY(r.u64("second-level scale count", &e.n_second));
        B2_TRY(r.u64("scale block size", &e.scale_block_size));
        uint32_t offset_bits = 0, flags = 0;
        B2_TRY(r.u32("scale offset", &offset_bits));
        B2_TRY(r.u32("flags", &flags));
        if (flags > 1u) return fail(B2_STATUS_INVALID_ARGUMENT, "packed model state has unknown flags");
        const bool dq = flags == 1u;
        if ((!dq && (e.n_scale_codes != 0 || e.n_second != 0 || e.scale_block_size != 0 || offset_bits != 0u)) ||
            (dq && (e.n_fp32_scales != 0 || e.scale_block_size == 0))) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "packed model state has inconsistent NF4 scale metadata");
        }
        std::memcpy(&e.offset, &offset_bits, sizeof(float));
        e.double_quantized = flags;
        // bytes this entry still needs: dims + the four arrays, with the reference's overflow rule
        uint64_t required = rank * sizeof(uint64_t);
        const uint64_t limit = std::numeric_limits<uint64_t>::max();
        const uint64_t counts[4] = {e.n_codes, e.n_fp32_scales, e.n_scale_codes, e.n_second};
        const uint64_t widths[4] = {1, sizeof(float), 1, sizeof(float)};
        for (int a = 0; a < 4; ++a) {
            if (counts[a] > (limit - required) / widths[a]) {
                return fail(B2_STATUS_OVERFLOW, "packed model state entry size exceeds addressable memory");
            }
            required += counts[a] * widths[a];
        }
        if (required > r.remaining()) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "truncated packed model state: weight payload");
        }
        B2_TRY(r.u64("dimension", &e.out_features));
        B2_TRY(r.u64("dimension", &e.in_features));
        B2_TRY(r.take(e.n_codes, "packed codes", &e.codes_offset));
        B2_TRY(r.take(e.n_fp32_scales * sizeof(float), "block scale", &e.fp32_scales_offset));
        if (dq) {
            B2_TRY(r.take(e.n_scale_codes, "scale codes", &e.scale_codes_offset));
            B2_TRY(r.take(e.n_second * sizeof(float), "second-level scale", &e.second_offset));
        }
        if (index < capacity) entries[index] = e;
    }
    if (r.remaining() != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "packed model state contains trailing bytes");
    }
    *count_out = count;
    return B2_STATUS_OK;
}
