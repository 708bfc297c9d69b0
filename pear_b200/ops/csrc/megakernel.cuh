// Layouts shared by the persistent decode megakernel (decode_megakernel.cu) and its host-side scheduler
// (pear_b200/deploy/schedule.py packs the same structs with `struct`).
//
// One launch runs one decode/verify step of a single sequence: every CTA (one per SM) walks its own instruction list.
// The role of upstream deploy/blackwell/nvfp4/csrc/megakernel.cu (`mk_main`, per-SM `Instr` lists of 32 B,
// common/csrc/step.cuh:8-16) re-derived for 148 SMs and sm_100a.
#pragma once
#include <stdint.h>

namespace mk {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one weight-streaming producer warp
constexpr int kTileRows = 128;                   // weight rows per stage (16 per consumer warp)
constexpr int kStageK = 256;                     // K elements per stage
constexpr int kStageCodeBytes = kTileRows * kStageK / 2;       // 16384: two e2m1 codes per byte
constexpr int kStageScaleBytes = kTileRows * kStageK / 16;     // 2048: one e4m3 scale per 16 elements
constexpr int kStageBytes = kStageCodeBytes + kStageScaleBytes;  // 18432
constexpr int kMaxSegStages = 20;                // activations of at most 20 * 256 = 5120 K elements sit in smem
constexpr int kXStride = kMaxSegStages * kStageK + 16;  // halves per token row; bytes = 32 mod 128 (bank spread)

enum Op : int {
  OP_END = 0,
  OP_GEMV = 1,          // a: row tile, b: first k-stage, c: k-stage count, d: flags (bit0: load activations)
  OP_BARRIER = 2,       // grid-wide barrier (every CTA's list holds the same number of them)
  OP_EMBED = 3,         // a: first column, b: column count
  OP_ZERO = 4,          // a: first float, b: float count
  OP_GDN = 5,           // a: value head, b: first row of the head, c: row count
  OP_ATTN = 6,          // a: kv head, b: split index, c: split count
  OP_ATTN_COMBINE = 7,  // a: first (row, q head) pair, b: pair count
  OP_SAMPLE_PART = 8,   // a: first vocab chunk, b: chunk count
  OP_SAMPLE_FIN = 9,    // run by one CTA: acceptance, next token, next step record
  OP_DRAFT_IN = 10,     // a: first column, b: column count: builds the drafter's fc input rows
  OP_ARGMAX_PART = 11,  // a: first vocab chunk, b: chunk count
  OP_ARGMAX_FIN = 12,   // run by one CTA: draft tokens into the next step record
  OP_COPY = 13,         // a: first float, b: float count: dst[i] = src[i]
  OP_QUANT = 14,        // a: first unit of 128 K elements, b: unit count: builds the next GEMV's activation operand
};

struct __align__(16) Instr {
  int32_t op, desc, a, b, c, d, e, f;
};
static_assert(sizeof(Instr) == 32, "Instr is 32 bytes");

enum Prologue : int { PRO_PLAIN = 0, PRO_NORM = 1, PRO_SWIGLU = 2, PRO_GDN_NORM = 3 };
enum Epilogue : int { EPI_RED = 0, EPI_STORE = 1 };

// Generic 128-byte op descriptor; the meaning of the fields depends on the op (see decode_megakernel.cu).
struct __align__(16) Desc {
  const void* p0;  // GEMV: packed weight stages          GDN: record rows (parity 0)    ATTN: q/k/v rows
  const void* p1;  // GEMV: input rows (fp32)              GDN: record rows (parity 1)    ATTN: k cache
  const void* p2;  // GEMV: norm weight / z rows           GDN: conv weight [C][4]        ATTN: v cache
  const void* p3;  // GEMV: gated-norm weight              GDN: A_log | dt_bias           ATTN: q_norm | k_norm weights
  void* p4;        // GEMV: output rows (fp32)             GDN: state slot                ATTN: partials
  void* p5;        //                                      GDN: conv slot                 ATTN: rope cos/sin table
  void* p6;        //                                      GDN: output rows
  void* p7;
  int32_t i0;      // GEMV: K                              GDN: record row stride         ATTN: row stride of q/k/v rows
  int32_t i1;      // GEMV: k-stages per tile              GDN: value heads               ATTN: kv heads
  int32_t i2;      // GEMV: real output rows
  int32_t i3;      // GEMV: input row stride (floats)
  int32_t i4;      // GEMV: output row stride (floats)
  int32_t i5;      // GEMV: prologue
  int32_t i6;      // GEMV: epilogue
  int32_t i7;      // flags: 1 input rows by parity (base + parity * i8 floats), 2 output by parity, 4 output by the
                   // other parity, 8 row count is the drafter's (rec_next->rows_draft) instead of rec->T
  int32_t i8;
  int32_t i9;
  float f0;        // GEMV: output scale (1 / global scale)
  float f1;        // eps
  float f2;
  float f3;
  int32_t pad[2];  // GEMV: [0] = 1 + descriptor of the GEMV whose operand this op's finishers build (0: none),
                   //       [1] = first of that link's tile counters
};
static_assert(sizeof(Desc) == 128, "Desc is 128 bytes");

// Per-sequence step record, on the device; the sampler/bookkeeping ops of step k write the record of step k + 1.
struct StepRec {
  int32_t T;          // rows of this step (1 + draft tokens), <= 8
  int32_t pos0;       // position of row 0 == number of tokens whose state is committed
  int32_t n_replay;   // rows of the previous block that were committed (GDN layers replay them first)
  int32_t parity;     // record parity of this step
  int32_t step;       // step counter (RNG stream, output ring slot)
  int32_t mode;       // 0 decode, 1 prefill (every row is committed, nothing is sampled)
  int32_t n_out_total;   // tokens emitted so far
  int32_t rows_draft; // rows the drafter runs in the launch that WRITES this record (committed rows + mask rows)
  int32_t tokens[8];  // row 0: the last emitted token; rows 1..: draft tokens
  int32_t n_acc;      // drafts accepted by the step that wrote this record
  int32_t aux[7];
};

// One slot of the output ring (device memory, copied to pinned host memory by the host per step).
struct StepOut {
  int32_t step, n_out, n_accept, pos0;
  int32_t tokens[8];
  float logprobs[4];
};

// Per-step control record the host copies from pinned memory before every launch: sampling parameters may change
// between steps of a session without rebuilding anything.
struct StepCtrl {
  float temperature;
  uint32_t seed;
  int32_t stop_token;   // -1: none (recorded in the output slot when emitted)
  int32_t reserved[5];
};

struct Params {
  const Instr* instrs;     // [num_ctas][max_instrs]
  const Desc* descs;
  StepRec* rec;            // [2]: rec[step & 1] is read, rec[(step + 1) & 1] is written
  StepOut* out_ring;       // [ring]
  uint32_t* barrier;       // grid barrier counter, monotonic across launches
  int* status;             // 0 = ok
  int32_t max_instrs;
  int32_t ring;
  int32_t step_parity;     // which rec is current
  uint32_t seed;
  float temperature;
  int32_t vocab;
  uint32_t barrier_base;   // value of the barrier counter when the launch starts (the counter is never reset)
  int32_t pad;
  const StepCtrl* ctrl;    // null: temperature/seed above
  // in-kernel tracing: CTAs below trace_ctas append (mark id, instruction index, globaltimer ns) records;
  // trace[cta * trace_cap] holds the record count, records follow (2 x uint64 each). Null: tracing off.
  unsigned long long* trace;
  int32_t trace_ctas;
  int32_t trace_cap;
  int32_t l2_ahead;        // weight stages the producer keeps requested into L2 beyond the shared-memory ring (0: off)
  int32_t pad2;
  int32_t* tile_cnt;           // arrival counters of the linked GEMVs' row tiles (zero between steps)
  const int32_t* tile_expect;  // instructions that contribute to each counter (per program)
};

}  // namespace mk
