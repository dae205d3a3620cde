// Host-side entry points of the kernels, one per translation unit; the C ABI and the runner call these.
#pragma once

#include "ts_common.cuh"

namespace ts {

bool skinny_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
size_t skinny_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, bool gated);
int linear_skinny(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                  int epilogue, float scale, int out_dtype, void *workspace, size_t workspace_bytes,
                  cudaStream_t stream);
bool umma_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
size_t umma_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, int epilogue);
int umma_take_status();
// Two-SM pairs (tcgen05 cta_group::2) on 256 x 256 tiles: prefill-sized m.
bool pair_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
struct StreamFused;
uint32_t pair_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue);  // partial sums per row it leaves, or 0
int linear_pair(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k, int epilogue,
                float scale, int out_dtype, cudaStream_t stream, const StreamFused *fused = nullptr);
int pair_take_status();
uint32_t pair_slots();  // SM pairs that can run the paired kernel at once
int linear_umma(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                int epilogue, float scale, int out_dtype, void *workspace, size_t workspace_bytes,
                cudaStream_t stream);
bool stream_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
int stream_take_status();
// The residual stream's RMS norms folded into the streamed linears on either side of them.
struct StreamFused {
    // In: x is bf16(row * gain) without the 1/rms factor, row_ss f32 [m, row_parts] are partial sums of squares
    // of the rows (any split that adds up to the row); the product's rows are multiplied by
    // 1/sqrt(sum/k + row_eps) before the epilogue.
    const float *row_ss = nullptr;
    uint32_t row_parts = 0;
    float row_eps = 0.0f;
    // Out: ss_out f32 [m, stream_sumsq_parts(...)] = per 128-column tile, the sum of squares of the finished
    // output rows; xs_out bf16 [m, n] = out * xs_gain[n], the next linear's x.
    float *ss_out = nullptr;
    void *xs_out = nullptr;
    const float *xs_gain = nullptr;
};
// Parts per row that a linear of this shape leaves in ss_out, or 0 when it cannot.
uint32_t stream_sumsq_parts(uint32_t m, uint32_t n, uint32_t k, int epilogue);
int linear_stream(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                  int epilogue, float scale, int out_dtype, cudaStream_t stream, const StreamFused *fused = nullptr);
// Picks the kernel family for a linear: TS_LINEAR_SKINNY, TS_LINEAR_STREAM, TS_LINEAR_UMMA, or -1.
int pick_linear_path(uint32_t m, uint32_t n, uint32_t k, int epilogue, int path);
size_t attend_rows_workspace_bytes(uint32_t rows, uint32_t keys, uint32_t heads, uint32_t kv_heads, uint32_t width);
// Fused front of the decode attention: q, k, v raw from the projection (qkv [rows, (heads + 2 kv_heads) * 128]
// bf16); the kernel norms and rotates q and k, appends k and v at kept_row(slot, position) and attends.
// Only where every row of the launch sits in a slot of its own (a decode step): a row must not read a
// key another row of the same launch appends.
struct RowsFused {
    const void *qkv = nullptr;
    const float *q_norm = nullptr, *k_norm = nullptr, *inv_freq = nullptr;
    float eps = 0.0f;
    // The kept rows, slots, positions and page table this launch reads were written two or more launches
    // ago: key and value tiles may be fetched before the upstream launch has completed.
    bool early_keys = false;
};
bool attend_rows_fused_supports(bool contiguous, uint32_t width, uint32_t kept_rows);
int attend_rows(const void *q, const void *k, const void *v, void *out, const uint32_t *slots,
                const uint32_t *positions, const KeptDev &kept, bool contiguous, uint32_t rows, uint32_t keys,
                uint32_t heads, uint32_t kv_heads, uint32_t width, uint32_t back, float scale, void *workspace,
                size_t workspace_bytes, cudaStream_t stream, uint32_t ahead = 0, const uint32_t *lens = nullptr,
                uint32_t kept_rows = 0,  // rows the K/V buffers hold; 0 = unknown
                const RowsFused *fused = nullptr);
int rows_take_status();
bool flash_supports(uint32_t width);
int flash_take_status();
int attend_flash(const void *q, const void *k, const void *v, void *out, const uint32_t *cu_seqlens, uint32_t seqs,
                 uint32_t queries, uint32_t keys, uint32_t total_q, uint32_t total_k, uint32_t heads, uint32_t kv_heads,
                 uint32_t width, uint32_t back, uint32_t ahead, float scale, cudaStream_t stream);
// Fills slots[r] = r / queries, positions[r] = past + r % queries for the rows fallback of whole attention.
int iota_rows(uint32_t *slots, uint32_t *positions, uint32_t seqs, uint32_t queries, uint32_t past, cudaStream_t stream);
int rms_norm(const void *x, int x_dtype, const float *w, void *out, int out_dtype, uint32_t rows, uint32_t width,
             float eps, const uint32_t *row_ids, cudaStream_t stream);
int gate(const volatile uint32_t *flag, cudaStream_t stream);
int mean_pool(const float *x, const uint32_t *cu_seqlens, float *out, uint32_t seqs, uint32_t width, int normalize,
              cudaStream_t stream);
int advance_rows(const uint32_t *ids, uint32_t *tokens, uint32_t *positions, uint32_t rows, cudaStream_t stream);
// Embedding rows as f32 plus xs = bf16(row * gain) and the rows' sums of squares (ss [rows, parts], all in part 0).
int gather_scaled(const void *table, const uint32_t *ids, float *out, void *xs, const float *gain, float *ss,
                  uint32_t parts, uint32_t rows, uint32_t table_rows, uint32_t width, cudaStream_t stream);
int gather_rows(const void *table, const uint32_t *ids, void *out, int out_dtype, uint32_t rows,
                uint32_t table_rows, uint32_t width, uint32_t first, cudaStream_t stream);
int scatter_rows(const void *x, const uint32_t *slots, const uint32_t *positions, void *out, const KeptDev &kept,
                 uint32_t rows, uint32_t width, cudaStream_t stream);
// k_dense, v_dense (optional): packed copies [rows, kv_heads, width] of the prepared keys and values.
int qk_norm_rope_append(const void *qkv, const float *q_norm, const float *k_norm, const float *inv_freq,
                        const uint32_t *slots, const uint32_t *positions, void *q_out, void *k_rows, void *v_rows,
                        const KeptDev &kept, uint32_t rows, uint32_t heads, uint32_t kv_heads, uint32_t width,
                        float eps, cudaStream_t stream, void *k_dense = nullptr, void *v_dense = nullptr);
size_t top_k_workspace_bytes(uint32_t rows, uint32_t width, uint32_t k);
int top_k(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, uint32_t k, void *workspace,
          size_t workspace_bytes, cudaStream_t stream);
int top_1_static(const void *x, int x_dtype, uint32_t *ids, uint32_t rows, uint32_t width, cudaStream_t stream);
int take_softmax(const float *x, const uint32_t *ids, float *gates, uint32_t rows, uint32_t width, uint32_t k,
                 cudaStream_t stream);


int moe_take_status();
size_t moe_workspace_bytes(uint32_t picks, uint32_t experts, uint32_t hidden, uint32_t ffn);
int moe_permutation(const uint32_t *ids, uint32_t *order, uint32_t *place, uint32_t *offsets, uint32_t *btiles,
                    uint32_t picks, uint32_t experts, uint32_t first, cudaStream_t stream);
int moe_experts(const void *x, const uint32_t *ids, const float *gates, const float *add, const void *w_in,
                const void *w_out, float *out, uint32_t picks, uint32_t repeat, uint32_t top, int mix, uint32_t experts,
                uint32_t first, uint32_t hidden, uint32_t ffn, void *workspace, size_t workspace_bytes,
                cudaStream_t stream);

int rope_angles(const uint32_t *positions, float *out, uint32_t count, uint32_t width, float theta, uint32_t turned,
                cudaStream_t stream);
int rope(void *x, int dtype, const float *freqs, uint32_t positions, uint32_t heads, uint32_t width, int adjacent,
         cudaStream_t stream);
bool plain_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
// Sequential f32 sums in ascending k, the interpreter's order: bit-exact scores for a router (no gated epilogue).
bool ordered_supports(uint32_t m, uint32_t n, uint32_t k, int epilogue);
int linear_ordered(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                   int epilogue, float scale, int out_dtype, cudaStream_t stream);
int linear_plain(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k,
                 int epilogue, float scale, int out_dtype, cudaStream_t stream);
size_t picked_workspace_bytes(uint32_t rows, uint32_t n, uint32_t k, uint32_t count);
int picked(const void *x, const void *w, const uint32_t *ids, float *out, uint32_t rows, uint32_t n, uint32_t k,
           uint32_t count, uint32_t stride, uint32_t offset, uint32_t repeat, uint32_t first, void *workspace,
           size_t workspace_bytes, cudaStream_t stream);
int moe_mix(const float *y_picks, const float *gates, const float *add, float *out, uint32_t rows, uint32_t top,
            uint32_t width, cudaStream_t stream);

// Decode-sized linear over Q8_0 weights (engine/ir/mem/src/block.rs:259-260) and the form's host-side packer.
bool q8_0_supports(uint32_t m, uint32_t n, uint32_t k);
size_t q8_0_workspace_bytes(uint32_t m, uint32_t n, uint32_t k);
int linear_q8_0(const void *x, const void *w, const void *a0, void *out, uint32_t m, uint32_t n, uint32_t k, int epilogue,
                float scale, int out_dtype, void *workspace, size_t workspace_bytes, cudaStream_t stream);
size_t q8_0_bytes(size_t elements);
void q8_0_pack(const float *data, size_t elements, uint8_t *out);
void q8_0_unpack(const uint8_t *bytes, size_t elements, float *out);

// The layer stack of a decode step (<= 64 rows, one per slot, head width 128) as one persistent kernel.
struct StepKernel;
struct StepKernelShape {
    uint32_t layers, hidden, heads, kv_heads, head_dim, ffn, vocab, page, kept_rows, max_rows;
    float eps;
    int qk_norm;
};
struct StepKernelLayer {
    const void *wqkv, *wo, *wgu, *wdown;
    const float *ln1, *ln2, *q_norm, *k_norm;
    void *k_rows, *v_rows;
};
struct StepKernelBuffers {
    const StepKernelLayer *layers;
    const void *embed;
    float *x;                 // residual rows f32 [max_rows, hidden]
    void *xs, *attn, *act;    // bf16 [max_rows, hidden | heads * 128 | ffn]
    void *qkv;                // bf16 [max_rows, (heads + 2 kv_heads) * 128]
    const uint32_t *tokens, *slots, *positions;
    const float *inv_freq;
};
bool step_kernel_supports(const StepKernelShape &shape);
uint32_t step_kernel_max_rows();
int step_kernel_create(const StepKernelShape &shape, const StepKernelBuffers &buffers, StepKernel **out);
void step_kernel_destroy(StepKernel *kernel);
// Gather + every layer for `rows` rows (tokens, slots, positions on the device) whose positions are all below
// `keys`; leaves the residual rows in x.
int step_kernel_launch(StepKernel *kernel, uint32_t rows, uint32_t keys, const KeptDev &kept, cudaStream_t stream);
int step_take_status();
// Runs a one-block kernel whose bounded wait runs out after `wait_ns`: the status word then reads TS_ERR_TIMEOUT.
int wait_runs_out(uint64_t wait_ns, cudaStream_t stream);

// Sets the process-wide programmatic-dependent-launch switch.
void set_pdl(bool enabled);

}  // namespace ts
