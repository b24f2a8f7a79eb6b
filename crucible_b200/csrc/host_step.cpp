// The step builder's inner part, native: packs the integer metadata of one step
// (token ids, positions, owners, wanted rows, per-request starts, lengths, slots and
// block tables) into the pinned block that one copy then takes to the device, and
// checks the tokens and wanted places on the way.  The layout is `StepLayout`'s
// (crucible_b200/engine/context.py): pieces in a fixed order, each padded to a
// multiple of four ints so that every piece starts on a 16-byte boundary.
//
// Host code only: no CUDA call is made here.  The reference builds the same arrays in
// its runtime (`engine/src/gpu_model.rs:2872-2896`: owners, positions, segments, final
// rows of a packed batch; `engine/src/runtime.rs:777-796`: tokens, positions, lengths
// and tables of a decode batch, rebuilt every step).
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define CB_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
inline int pad4(int n) { return (n + 3) / 4 * 4; }
}

// Offsets of the pieces for a step of n_tokens rows, n_req requests and n_want wanted
// rows with n_groups block tables of the given strides.  offsets: 8 + n_groups + 1 ints
// (token_ids, positions, row_request, logit_rows, req_row_start, req_context_len,
// req_first_pos, req_state_slot, table0.., total).
CB_EXPORT void cb_host_step_offsets(int n_tokens, int n_req, int n_want, int n_groups,
                                    const int32_t* strides, int32_t* offsets) {
    int at = 0, i = 0;
    const int sizes[8] = {n_tokens, n_tokens, n_tokens, n_want, n_req + 1, n_req, n_req, n_req};
    for (; i < 8; ++i) {
        offsets[i] = at;
        at += pad4(sizes[i]);
    }
    for (int g = 0; g < n_groups; ++g) {
        offsets[i++] = at;
        at += pad4(n_req * strides[g]);
    }
    offsets[i] = at;
}

// tokens: the step's tokens, request after request; a request whose only token is
// `device_token` means "the token last chosen for this request, kept on the device":
// its id goes out as -(slot + 1).  wants: places among each request's own tokens,
// ascending.  rows: n_groups * n_req pointers (group-major) to the requests' table rows
// of `strides[g]` ints each.  Returns 0, or a code with a message in `err`:
// 1 a request brings no tokens, 2 a token outside the vocabulary, 3 a context too long,
// 4 a wanted place outside the request's tokens, 5 wanted places not ascending.
CB_EXPORT int cb_host_pack_step(int32_t* dst, int n_req, const int32_t* counts,
                                const int32_t* first_pos, const int32_t* slots,
                                const int64_t* tokens, const int32_t* want_counts,
                                const int32_t* wants, int n_groups, const int32_t* strides,
                                const int32_t* const* rows, int vocab, int max_context,
                                long long device_token, int32_t* bad_request, char* err,
                                int err_len) {
    int n_tokens = 0, n_want = 0;
    for (int r = 0; r < n_req; ++r) {
        if (counts[r] <= 0) {
            *bad_request = r;
            snprintf(err, err_len, "brings no tokens");
            return 1;
        }
        n_tokens += counts[r];
        n_want += want_counts[r];
    }
    int32_t off[8 + 64 + 1];
    if (n_groups > 64) n_groups = 64;
    cb_host_step_offsets(n_tokens, n_req, n_want, n_groups, strides, off);
    int32_t* token_ids = dst + off[0];
    int32_t* positions = dst + off[1];
    int32_t* row_request = dst + off[2];
    int32_t* logit_rows = dst + off[3];
    int32_t* req_row_start = dst + off[4];
    int32_t* req_context_len = dst + off[5];
    int32_t* req_first_pos = dst + off[6];
    int32_t* req_state_slot = dst + off[7];
    int row = 0, w = 0;
    for (int r = 0; r < n_req; ++r) {
        const int n = counts[r];
        if (first_pos[r] + n > max_context) {
            *bad_request = r;
            snprintf(err, err_len, "would hold %d tokens; the model's context is %d",
                     first_pos[r] + n, max_context);
            return 3;
        }
        req_row_start[r] = row;
        req_first_pos[r] = first_pos[r];
        req_context_len[r] = first_pos[r] + n;
        req_state_slot[r] = slots[r];
        if (n == 1 && tokens[row] == device_token) {
            token_ids[row] = -(slots[r] + 1);
            positions[row] = first_pos[r];
            row_request[row] = r;
        } else {
            for (int i = 0; i < n; ++i) {
                const long long t = tokens[row + i];
                if (t < 0 || t >= vocab) {
                    *bad_request = r;
                    snprintf(err, err_len, "token %lld is outside the vocabulary of %d", t, vocab);
                    return 2;
                }
                token_ids[row + i] = (int32_t)t;
                positions[row + i] = first_pos[r] + i;
                row_request[row + i] = r;
            }
        }
        int last = -1;
        for (int i = 0; i < want_counts[r]; ++i) {
            const int place = wants[w + i];
            if (place < 0 || place >= n) {
                *bad_request = r;
                snprintf(err, err_len, "wanted place %d is outside its %d tokens", place, n);
                return 4;
            }
            if (place <= last) {
                *bad_request = r;
                snprintf(err, err_len, "wanted places must ascend");
                return 5;
            }
            last = place;
            logit_rows[w + i] = row + place;
        }
        w += want_counts[r];
        row += n;
    }
    req_row_start[n_req] = row;
    for (int g = 0; g < n_groups; ++g) {
        int32_t* block = dst + off[8 + g];
        const int stride = strides[g];
        for (int r = 0; r < n_req; ++r)
            memcpy(block + (size_t)r * stride, rows[(size_t)g * n_req + r], (size_t)stride * sizeof(int32_t));
    }
    return 0;
}
