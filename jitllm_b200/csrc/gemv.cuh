// Decode-time quantised matrix-vector product: interface between the engine and gemv.cu, and the
// work partition both the kernel and its host-side checks use.
#pragma once

#include "formats.cuh"
#include "tp_exchange.cuh"

namespace jl {

// One weight matrix of a fused launch (Q, K and V share one launch; gate and up share one).
struct GemvSeg {
    const uint8_t *w;  // device, GGUF block layout (Q6_K: the copy with padded super-blocks), rows x cols, 16-byte aligned
    float *y;          // device, rows
    const float *res;  // nullable: y[row] = res[row] + dot (may alias y)
    int rows;
};

enum GemvMode : int { kGemvPlain = 0, kGemvGateUp = 1 };

// Tensor parallelism: the all-reduce that follows a row-parallel projection (output projection, down
// projection), done by the mat-vec's own epilogue over peer memory. Every rank cuts its rows into
// the same CTA ranges; the thread that finishes row r on this GPU stores its partial sum into every
// peer's inbox, collects the peers' partial sums of the same row from its own inbox, adds them in
// rank order (every GPU gets the same bits) to the residual and writes the row. tp == 0: off.
struct GemvTpReduce {
    TpInboxes inbox;
    size_t base, cap;   // the reduce region of an inbox and its packets per (slot, source rank)
    int tp, rank;
    int row_offset;     // index of this launch's row 0 inside that region (batch row * dim)
    unsigned *ctr;      // [0] sequence of this exchange, [1] CTA arrivals; advanced by the last CTA
    unsigned long long timeout_ns;
};

struct GemvArgs {
    GemvSeg seg[3];
    int nseg;
    int cols;  // multiple of 256, at most kGemvMaxCols
    int type;  // kQ8_0 / kQ4_0 / kQ4_K, or kQ6_K where gemv_takes() says so
    int mode;
    const float *x;       // cols floats, 16-byte aligned
    const float *norm_w;  // nullable: y = W . (norm_w * (rsqrt(mean(x^2)+eps) * x))
    float eps;
    const uint8_t *active;  // nullable: a zero byte turns the whole launch into a no-op
    // Greedy argmax over the rows of seg[0] fused into the epilogue (nullable = off).
    float *argmax_val;       // gridDim.x partial maxima
    int *argmax_idx;         // gridDim.x partial indices
    unsigned *argmax_count;  // zero on entry, zero again on exit
    int *out_token;
    int *status;  // device status word, see common.cuh
    GemvTpReduce tpr;  // plain launches of one matrix with a residual only
};

// Geometry of one launch. A CTA has 16 consumer warps and one producer warp. A row is cut into
// chunks of 2048 columns; consumer warp w works on chunk w % nchunks of the rows of group
// w / nchunks and keeps that chunk of the activation in registers for the whole launch. The warps
// of a group share one ring of stages; a stage holds whole rows, fetched by one bulk copy (copies
// of 4 KB and more are what reaches the HBM rate; 1 KB copies reach half of it).
constexpr int kGemvConsumerWarps = 16;
constexpr int kGemvThreads = (kGemvConsumerWarps + 1) * 32;
constexpr int kGemvChunkCols = 2048;
constexpr int kGemvMaxCols = kGemvConsumerWarps * kGemvChunkCols;
constexpr int kGemvMaxStages = 12;

struct GemvPlan {
    int grid;
    size_t smem_bytes;
    int nchunks;        // chunks per row = consumer warps that share a row
    int groups;         // row groups per CTA; groups * nchunks <= 16
    int stages;         // ring depth per group
    int phase_jobs;     // jobs (rows, or gate/up pairs) a group handles between two epilogues
    int off_x;          // shared-memory offsets: activation planes,
    int off_partial;    //   per-chunk partial sums [nchunks][groups * phase_jobs * streams per job],
    int off_ring;       //   weight rings [groups][stages][rows per stage * row bytes]
};

// Jobs (rows, or gate/up row pairs) are dealt to CTAs, and inside a CTA to groups, as contiguous
// ranges of near-equal length.
__host__ __device__ inline int gemv_split(int n, int part, int parts) {
    return static_cast<int>(static_cast<long long>(n) * part / parts);
}
// Rows per stage (a stage is one bulk copy of whole consecutive rows, completing on one mbarrier
// phase): two for the 4-bit formats, one for Q8_0 whose rows are twice as long in bytes.
__host__ __device__ inline int gemv_rows_per_stage(int type) { return type == kQ8_0 ? 1 : 2; }  // = Fmt<type>::streams

// The formats this kernel reads: Q8_0, Q4_0, Q4_K, Q4_1, Q5_K, and Q6_K from its padded copy (rows are fetched by bulk
// copies and must be whole 16-byte pieces: 210-byte super-blocks are not, kQ6_KPadded-byte ones are).
__host__ __device__ inline bool gemv_takes(int type, int64_t cols) {
    if (cols <= 0 || cols % 256 != 0) return false;
    return is_quant(type) || type == kQ6_K || type == kQ5_K || type == kQ4_1;
}
// Bytes of one matrix row as this kernel reads it.
__host__ __device__ inline int64_t gemv_row_bytes(int type, int64_t cols) {
    return type == kQ6_K ? cols / 256 * kQ6_KPadded : row_bytes(type, cols);
}

// Chooses group count, pipeline depth and shared-memory layout for one launch shape.
bool gemv_plan(int type, int cols, int total_rows, int mode, int sm_count, GemvPlan *out);
// Sets the dynamic shared memory attribute of every instantiation; once per process per device.
cudaError_t gemv_configure();
cudaError_t gemv_launch(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream,
                        bool programmatic);
cudaError_t gemv_trace_bind(unsigned long long *buf, unsigned cap, int mode);

// The activation is split into this many signed 8-bit digits before the integer dot products:
// x ~ s_blk * (256 * a1 + a2) with one scale per 32 elements, so |x - approx| <= s_blk / 2 with
// s_blk = max|x| / kDigitRange: a 16-bit fixed-point activation per block.
constexpr int kDigits = 2;
constexpr float kDigitRange = 32639.0f;  // 127 * 256 + 127

}  // namespace jl
