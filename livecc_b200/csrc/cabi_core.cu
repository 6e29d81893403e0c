// C-ABI entry points every model family needs: context, launch counter, the tensor-core GEMM and token selection.
// Kept apart from cabi.cu so that a library holding only one model family's kernels can be linked.
#include "../../include/livecc_b200.h"
#include "cabi_common.h"
#include "gemm.h"
#include "launch.h"
#include "ops.h"

using lcc::bf16;

extern "C" {

int lcc_abi_version(void) { return LCC_ABI_VERSION; }

lcc_ctx* lcc_create(int device) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return nullptr;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return nullptr;
    if (prop.major != 10) return nullptr;  // sm_100a only: there is no fallback path
    if (cudaSetDevice(device) != cudaSuccess) return nullptr;
    lcc_ctx* c = new lcc_ctx();
    c->device = device;
    c->num_sms = prop.multiProcessorCount;
    c->err[0] = 0;
    return c;
}

void lcc_destroy(lcc_ctx* ctx) { delete ctx; }

const char* lcc_last_error(lcc_ctx* ctx) { return ctx ? ctx->err : "null ctx"; }

int lcc_num_sms(lcc_ctx* ctx) { return ctx ? ctx->num_sms : -1; }

uint64_t lcc_launch_count(void) { return lcc::g_launches.load(std::memory_order_relaxed); }

int lcc_gemm_bf16(lcc_ctx* ctx, const void* A, int lda, const void* B, int ldb, void* C, int ldc,
                  int M, int N, int K, const void* bias, const void* residual, int ldr, int epilogue,
                  int block_n, void* splitk_ws, int64_t splitk_ws_bytes, lcc_stream_t stream) {
    if (!ctx) return -1;
    lcc::GemmArgs a;
    a.splitk_ws = splitk_ws;
    a.splitk_ws_bytes = splitk_ws_bytes > 0 ? (size_t)splitk_ws_bytes : 0;
    a.A = A; a.B = B; a.C = C;
    a.M = M; a.N = N; a.K = K;
    a.lda = lda; a.ldb = ldb; a.ldc = ldc;
    a.bias = bias; a.residual = residual; a.ldr = ldr;
    a.epi = epilogue; a.block_n = block_n;
    int r = lcc::gemm_bf16_tn(a, ctx->num_sms, (cudaStream_t)stream);
    if (r) LCC_FAIL(ctx, r, "lcc_gemm_bf16 failed (code %d; M=%d N=%d K=%d epi=%d)", r, M, N, K, epilogue);
    return 0;
}


#define OP_RET(ctx, expr, name)                                              \
    do {                                                                     \
        if (!(ctx)) return -1;                                               \
        int rc__ = (expr);                                                   \
        if (rc__) LCC_FAIL(ctx, rc__, name " failed (code %d)", rc__);       \
        LCC_CHECK_LAUNCH(ctx, name);                                         \
        return 0;                                                            \
    } while (0)

int lcc_sample_greedy(lcc_ctx* ctx, const float* logits_raw, float* logits_proc, int V, int64_t* seq,
                      int32_t* scalars, const lcc_sampling* sp, int advance_kv, const void* embed, void* h,
                      int H, lcc_stream_t stream) {
    if (!sp) return -1;
    lcc::SampleArgs a{};
    a.logits_raw = logits_raw; a.logits_proc = logits_proc; a.V = V; a.seq = seq; a.scalars = scalars;
    a.repetition_penalty = sp->repetition_penalty; a.inv_repetition_penalty = sp->inv_repetition_penalty; a.thr_token = sp->thr_token; a.thr_base = sp->thr_base;
    a.thr_step = sp->thr_step; a.eos_token_id = sp->eos_token_id; a.eos_token_id2 = sp->eos_token_id2;
    a.max_new_tokens = sp->max_new_tokens;
    a.advance_kv = advance_kv; a.embed = (const bf16*)embed; a.h = (bf16*)h; a.H = H;
    OP_RET(ctx, lcc::sample_greedy(a, (cudaStream_t)stream), "lcc_sample_greedy");
}

}  // extern "C"
