// extern "C" entry points of libmlstm_b200.so (declared in include/mlstm_b200.h): argument checks,
// workspace carving and the launch sequences.  Nothing here allocates or synchronises.
#include <cmath>
#include <cstdio>
#include <mutex>

#include "mlstm_common.cuh"

namespace mlstm {
namespace {

constexpr size_t WS_ALIGN = 256;
constexpr size_t al(size_t x) { return (x + WS_ALIGN - 1) / WS_ALIGN * WS_ALIGN; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool dtype_ok(int dt) { return dt == MLSTM_DT_F32 || dt == MLSTM_DT_F16 || dt == MLSTM_DT_BF16; }

struct Carver {
    uint8_t* base;
    size_t off = 0;
    explicit Carver(void* b) : base(static_cast<uint8_t*>(b)) {}
    template <typename T>
    T* take(size_t bytes) {
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += al(bytes);
        return p;
    }
};

struct FwdWs {
    int* status;
    float *ga, *gAn, *gaw, *m, *b;
    double *a_ref, *An_ref;
    size_t bytes;
};
// Byte offsets of the forward scratch, usable at compile time (the built-in scratch of
// mlstm_forward_f16_static is sized from it).  with_mb: also m and b (entry points whose caller does not pass them).
struct FwdLayout {
    size_t ga, gAn, gaw, a_ref, An_ref, m, b, bytes;
};
constexpr FwdLayout fwd_layout(size_t BH, size_t S, bool with_mb) {
    FwdLayout l{};
    const size_t spad = (S + TILE - 1) / TILE * TILE;
    const size_t vec = BH * spad * sizeof(float);
    size_t off = WS_ALIGN;   // status word and work-item counters
    l.ga = off; off += al(vec);
    l.gAn = off; off += al(vec);
    l.gaw = off; off += al(vec);
    l.a_ref = off; off += al(vec / REF_BLOCK * 2);
    l.An_ref = off; off += al(vec / REF_BLOCK * 2);
    l.m = off;
    if (with_mb) off += al(BH * S * sizeof(float));
    l.b = off;
    if (with_mb) off += al(BH * S * sizeof(float));
    l.bytes = off;
    return l;
}
FwdWs carve_fwd(void* ws, int BH, int S, bool with_mb) {
    const FwdLayout l = fwd_layout(static_cast<size_t>(BH), static_cast<size_t>(S), with_mb);
    uint8_t* base = static_cast<uint8_t*>(ws);
    FwdWs w{};
    w.bytes = l.bytes;
    if (!base) return w;
    w.status = reinterpret_cast<int*>(base);
    w.ga = reinterpret_cast<float*>(base + l.ga);
    w.gAn = reinterpret_cast<float*>(base + l.gAn);
    w.gaw = reinterpret_cast<float*>(base + l.gaw);
    w.a_ref = reinterpret_cast<double*>(base + l.a_ref);
    w.An_ref = reinterpret_cast<double*>(base + l.An_ref);
    if (with_mb) {
        w.m = reinterpret_cast<float*>(base + l.m);
        w.b = reinterpret_cast<float*>(base + l.b);
    }
    return w;
}

struct BwdWs {
    int* status;
    float *ga, *gAn, *gaw, *gB, *gBw, *g, *dI, *R;
    double *a_ref, *An_ref;
    void* dh16;
    size_t bytes;
};
BwdWs carve_bwd(void* ws, int BH, int S, int D, bool need_dh16) {
    Carver c(ws);
    BwdWs w{};
    const size_t vec = static_cast<size_t>(BH) * round_up(S, TILE) * sizeof(float);
    w.status = c.take<int>(WS_ALIGN);
    w.ga = c.take<float>(vec);
    w.gAn = c.take<float>(vec);
    w.a_ref = c.take<double>(vec / REF_BLOCK * 2);
    w.An_ref = c.take<double>(vec / REF_BLOCK * 2);
    w.gaw = c.take<float>(vec);
    w.gB = c.take<float>(vec);
    w.gBw = c.take<float>(vec);
    w.g = c.take<float>(vec);
    w.dI = c.take<float>(vec * TC_DOT_PARTS);   // partial row dots, one per gate group of the tensor-core passes
    w.R = c.take<float>(vec * TC_DOT_PARTS);
    w.dh16 = need_dh16 ? c.take<uint8_t>(static_cast<size_t>(BH) * S * D * 2) : nullptr;
    w.bytes = c.off;
    return w;
}

int check_dims(int B, int NH, int S, int D) {
    if (B <= 0 || NH <= 0 || S <= 0 || D <= 0) return MLSTM_E_ARG;
    if (static_cast<long long>(B) * NH > 65535) return MLSTM_E_SHAPE;
    if (D % 8 != 0) return MLSTM_E_SHAPE;  // rows must stay 16-byte aligned for vector access
    if (static_cast<long long>(B) * NH * round_up(S, TILE) > 0x7fffffffLL / 32) return MLSTM_E_SHAPE;
    return MLSTM_OK;
}

// How a pass runs.  fp32 inputs: IEEE fp32 on the CUDA cores when forced or when no tensor-core form applies;
// single tf32 products only when the caller allows that arithmetic; otherwise, for D = 64 and 128, the
// split form (three bf16 products per fp32 product, fp32 accumulate) whose error is at fp32 level.
enum PassKind { KIND_SIMT = 0, KIND_TC = 1, KIND_TC_X3 = 2 };

int pass_kind(int S, int D, int dtype, int flags, int* rc) {
    *rc = MLSTM_OK;
    if ((flags & MLSTM_F_FORCE_SIMT) && (flags & MLSTM_F_FORCE_TC)) {
        *rc = MLSTM_E_ARG;
        return KIND_SIMT;
    }
    int kind = KIND_SIMT;
    if (dtype != MLSTM_DT_F32) {
        if (tc_supported(S, D, dtype)) kind = KIND_TC;
    } else if ((flags & MLSTM_F_ALLOW_TF32) && tc_supported(S, D, dtype)) {
        kind = KIND_TC;
    } else if (!(flags & MLSTM_F_NO_SPLIT) && tc_x3_supported(S, D)) {
        kind = KIND_TC_X3;
    }
    if (flags & MLSTM_F_FORCE_SIMT) return KIND_SIMT;
    if ((flags & MLSTM_F_FORCE_TC) && kind == KIND_SIMT) *rc = MLSTM_E_UNSUPPORTED;
    return kind;
}

// fp32 inputs on the tensor cores work on converted copies of the operands in the workspace (n tensors):
// tf32-rounded fp32 copies, or bf16 hi | mid copies of the same size.
size_t tf32_copy_bytes(int BH, int S, int D, int dtype, int flags, int ntensors) {
    int rc;
    const int kind = pass_kind(S, D, dtype, flags, &rc);
    return (dtype == MLSTM_DT_F32 && kind != KIND_SIMT) ? ntensors * al(static_cast<size_t>(BH) * S * D * sizeof(float)) : 0;
}
// converts `count` tensors into consecutive regions of `buf` and redirects the pointers
int round_inputs(const void** ptrs, int count, void* buf, int BH, int S, int D, int kind, cudaStream_t st) {
    const size_t one = al(static_cast<size_t>(BH) * S * D * sizeof(float));
    if (kind == KIND_TC_X3 && count <= 4) {   // one launch for all of them
        void* dst[4];
        for (int k = 0; k < count; k++) dst[k] = static_cast<uint8_t*>(buf) + k * one;
        int rc = launch_split_bf16_multi(ptrs, dst, count, static_cast<long long>(BH) * S, D, st);
        if (rc != MLSTM_OK) return rc;
        for (int k = 0; k < count; k++) ptrs[k] = dst[k];
        return MLSTM_OK;
    }
    for (int k = 0; k < count; k++) {
        void* dst = static_cast<uint8_t*>(buf) + k * one;
        int rc = kind == KIND_TC_X3 ? launch_split_bf16(ptrs[k], dst, static_cast<long long>(BH) * S, D, st)
                                    : launch_round_tf32(ptrs[k], dst, static_cast<long long>(BH) * S * D, st);
        if (rc != MLSTM_OK) return rc;
        ptrs[k] = dst;
    }
    return MLSTM_OK;
}

int run_pass(int kind, int mode, const PassParams& p, int in_dt, int out_dt, cudaStream_t st) {
    if (kind == KIND_TC_X3) return launch_pass_tc_x3(mode, p, st);
    return kind == KIND_TC ? launch_pass_tc(mode, p, in_dt, out_dt, st) : launch_pass_simt(mode, p, in_dt, out_dt, st);
}

int forward_impl(const void* q, const void* k, const void* v, const void* f, const void* i, const void* o, void* h,
                 float* m, float* b, const FwdWs& w, int BH, int S, int D, int dtype, int h_dtype, int flags,
                 cudaStream_t st, void* tf32buf = nullptr) {
    int rc;
    const int kind = pass_kind(S, D, dtype, flags, &rc);
    if (rc != MLSTM_OK) return rc;
    const int Spad = round_up(S, TILE);
    // (the gate pass also clears the status word and the passes' work-item counters)
    if ((rc = launch_gates_fwd(f, i, w.ga, w.gAn, w.a_ref, w.An_ref, m, BH, S, Spad, dtype, st, nullptr, nullptr, nullptr, 0, nullptr,
                               w.gaw, w.status, STATUS_WORDS)) != MLSTM_OK)
        return rc;
    const void* in[3] = {q, k, v};
    if (kind != KIND_SIMT && dtype == MLSTM_DT_F32) {
        if (!tf32buf) return MLSTM_E_WORKSPACE;
        if ((rc = round_inputs(in, 3, tf32buf, BH, S, D, kind, st)) != MLSTM_OK) return rc;
    }
    PassParams p{};
    p.S = S; p.Spad = Spad; p.BH = BH; p.D = D;
    p.X = in[0]; p.Y = in[1]; p.Z = in[2];
    p.row_rel = w.gAn; p.row_ref = w.An_ref; p.col_rel = w.ga; p.col_w = w.gaw; p.col_ref = w.a_ref;
    p.er_add = -0.5f * log2f(static_cast<float>(D));
    p.out = h; p.m = m; p.b_out = b; p.ogate = o;
    p.status = w.status; p.sched = w.status + 8; p.sched_zeroed = 1;
    return run_pass(kind, FWD, p, dtype, h_dtype, st);
}

// Two-pass forward for head dimensions above 256 (scan_gemm.cu): gates, W = gate(Q K^T) into scratch, h = (W V) / n
// (times silu(o) when o is given).  `extra` points behind the gate vectors of `w`: row-sum partials, then W.
size_t two_pass_extra_bytes(int BH, int S, int dtype) {
    return al(scan_gemm_bpart_bytes(BH, S, dtype)) + al(scan_gemm_w_bytes(BH, S, dtype));
}

int two_pass_forward(const void* q, const void* k, const void* v, const void* f, const void* i, const void* o, float* h,
                     float* m, float* b, const FwdWs& w, uint8_t* extra, int BH, int S, int D, int dtype, cudaStream_t st) {
    const int Spad = round_up(S, TILE);
    float* bpart = reinterpret_cast<float*>(extra);
    void* W = extra + al(scan_gemm_bpart_bytes(BH, S, dtype));
    // the gate pass clears the status word and the work-item counters of the two passes
    int rc;
    if ((rc = launch_gates_fwd(f, i, w.ga, w.gAn, w.a_ref, w.An_ref, m, BH, S, Spad, dtype, st, nullptr, nullptr, nullptr, 0,
                               nullptr, w.gaw, w.status, STATUS_WORDS)) != MLSTM_OK)
        return rc;
    ScanGemmArgs a{};
    a.S = S; a.Spad = Spad; a.BH = BH; a.D = D;
    a.ga = w.ga; a.gAn = w.gAn; a.gaw = w.gaw; a.a_ref = w.a_ref; a.An_ref = w.An_ref; a.m = m; a.b = b;
    a.bpart = bpart; a.status = w.status; a.counters = w.status + 8 + 12;
    return launch_scan_gemm(q, k, v, o, h, W, a, dtype, st);
}

// The parallel forward's own use of the two-pass form: head dimension above 256, float32 h, and for float32 inputs
// only where single tf32 products are allowed.
bool mm_fwd_two_pass(int S, int D, int dtype, int h_dtype, int flags) {
    if (flags & (MLSTM_F_FORCE_SIMT | MLSTM_F_FORCE_TC)) return false;
    if (h_dtype != MLSTM_DT_F32) return false;
    if (dtype == MLSTM_DT_F32 && !(flags & MLSTM_F_ALLOW_TF32)) return false;
    return scan_gemm_supported(S, D, dtype);
}

// The parallel backward's use of the same two passes: head dimension above 256, any h type, and for float32
// inputs only where single tf32 products are allowed.
bool mm_bwd_two_pass(int S, int D, int dtype, int flags) {
    if (flags & (MLSTM_F_FORCE_SIMT | MLSTM_F_FORCE_TC)) return false;
    if (dtype == MLSTM_DT_F32 && !(flags & MLSTM_F_ALLOW_TF32)) return false;
    return scan_gemm_supported(S, D, dtype);
}

// behind the gate vectors: the two gated matrices of a group of slices, then the row-dot partials R and dI
// (one per 256-column output slice)
size_t two_pass_bwd_extra_bytes(int BH, int S, int D, int dtype) {
    const size_t vec = static_cast<size_t>(BH) * round_up(S, TILE) * sizeof(float);
    return 2 * al(scan_gemm_bwd_matrix_bytes(BH, S, dtype)) + 2 * al(vec * (D / 256));
}

}  // namespace

static thread_local char g_error_detail[256] = "";
int note_cuda_error(cudaError_t err, const char* where) {
    snprintf(g_error_detail, sizeof(g_error_detail), "%s: %s (%s)", where, cudaGetErrorString(err), cudaGetErrorName(err));
    return MLSTM_E_CUDA;
}
}  // namespace mlstm

using namespace mlstm;

extern "C" {

const char* mlstm_status_string(int s) {
    switch (s) {
        case MLSTM_OK: return "ok";
        case MLSTM_E_ARG: return "bad argument (null pointer, non-positive size, unknown dtype or flag)";
        case MLSTM_E_SHAPE: return "shape not accepted (D must be a multiple of 8; B*NH <= 65535)";
        case MLSTM_E_ALIGN: return "tensor pointer not 16-byte aligned";
        case MLSTM_E_UNSUPPORTED: return "tensor-core path demanded for an unsupported case";
        case MLSTM_E_WORKSPACE: return "workspace missing or too small";
        case MLSTM_E_CUDA: return "CUDA runtime or driver call failed";
        case MLSTM_E_TIMEOUT: return "a kernel gave up on an internal wait";
        case MLSTM_E_STATIC_LIMIT:
            return "sequence too long for the built-in scratch of mlstm_forward_f16_static (S <= 16384); "
                   "use mlstm_forward_f16 with a workspace";
    }
    return "unknown status";
}

const char* mlstm_last_error_detail(void) { return g_error_detail; }

int mlstm_tc_supported(int S, int D, int dtype) {
    if (!tc_supported(S, D, dtype)) return 0;
    return dtype == MLSTM_DT_F32 ? 2 : 1;
}

size_t mlstm_mm_fwd_workspace(int B, int NH, int S, int D, int dtype, int flags) {
    if (check_dims(B, NH, S, D) != MLSTM_OK) return 0;
    // (sized for float32 h; a 16-bit h at these head dimensions takes the smaller one-pass workspace)
    if (mm_fwd_two_pass(S, D, dtype, MLSTM_DT_F32, flags))
        return carve_fwd(nullptr, B * NH, S, false).bytes + two_pass_extra_bytes(B * NH, S, dtype);
    return carve_fwd(nullptr, B * NH, S, false).bytes + tf32_copy_bytes(B * NH, S, D, dtype, flags, 3);
}

int mlstm_mm_fwd(const void* q, const void* k, const void* v, const void* f, const void* i, void* h, float* m, float* b,
                 void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int h_dtype, int flags,
                 void* stream) {
    if (!q || !k || !v || !f || !i || !h || !m || !b) return MLSTM_E_ARG;
    if (!dtype_ok(dtype) || (h_dtype != MLSTM_DT_F32 && h_dtype != dtype)) return MLSTM_E_ARG;
    int rc = check_dims(B, NH, S, D);
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(h)) return MLSTM_E_ALIGN;
    FwdWs w = carve_fwd(workspace, B * NH, S, false);
    if (mm_fwd_two_pass(S, D, dtype, h_dtype, flags)) {
        if (!workspace || workspace_bytes < w.bytes + two_pass_extra_bytes(B * NH, S, dtype) || !aligned16(workspace))
            return MLSTM_E_WORKSPACE;
        return two_pass_forward(q, k, v, f, i, nullptr, static_cast<float*>(h), m, b, w, static_cast<uint8_t*>(workspace) + w.bytes,
                                B * NH, S, D, dtype, static_cast<cudaStream_t>(stream));
    }
    const size_t extra = tf32_copy_bytes(B * NH, S, D, dtype, flags, 3);
    if (!workspace || workspace_bytes < w.bytes + extra || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    return forward_impl(q, k, v, f, i, nullptr, h, m, b, w, B * NH, S, D, dtype, h_dtype, flags,
                        static_cast<cudaStream_t>(stream), extra ? static_cast<uint8_t*>(workspace) + w.bytes : nullptr);
}

size_t mlstm_mm_bwd_workspace(int B, int NH, int S, int D, int dtype, int h_dtype, int flags) {
    if (check_dims(B, NH, S, D) != MLSTM_OK) return 0;
    if (mm_bwd_two_pass(S, D, dtype, flags))
        return carve_bwd(nullptr, B * NH, S, D, dtype != MLSTM_DT_F32 && h_dtype != dtype).bytes +
               two_pass_bwd_extra_bytes(B * NH, S, D, dtype);
    return carve_bwd(nullptr, B * NH, S, D, dtype != MLSTM_DT_F32 && h_dtype != dtype).bytes +
           tf32_copy_bytes(B * NH, S, D, dtype, flags, 4);
}

int mlstm_mm_bwd(const void* dh, const void* q, const void* k, const void* v, const void* f, const void* i, const void* h,
                 const float* m, const float* b, void* dq, void* dk, void* dv, void* df, void* di, void* workspace,
                 size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int h_dtype, int flags, void* stream) {
    if (!dh || !q || !k || !v || !f || !i || !h || !m || !b || !dq || !dk || !dv || !df || !di) return MLSTM_E_ARG;
    if (!dtype_ok(dtype) || (h_dtype != MLSTM_DT_F32 && h_dtype != dtype)) return MLSTM_E_ARG;
    int rc = check_dims(B, NH, S, D);
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(dh) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(h) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return MLSTM_E_ALIGN;
    const int BH = B * NH, Spad = round_up(S, TILE);
    const bool need16 = dtype != MLSTM_DT_F32 && h_dtype != dtype;
    BwdWs w = carve_bwd(workspace, BH, S, D, need16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mm_bwd_two_pass(S, D, dtype, flags)) {
        if (!workspace || workspace_bytes < w.bytes + two_pass_bwd_extra_bytes(BH, S, D, dtype) || !aligned16(workspace))
            return MLSTM_E_WORKSPACE;
        // the gate pass clears the status word and the work-item counters of the five launches
        if ((rc = launch_gates_fwd(f, i, w.ga, w.gAn, w.a_ref, w.An_ref, nullptr, BH, S, Spad, dtype, st, nullptr, nullptr, nullptr,
                                   0, nullptr, w.gaw, w.status, STATUS_WORDS)) != MLSTM_OK)
            return rc;
        if ((rc = launch_bwd_prep(h, dh, b, m, w.gAn, w.gB, w.gBw, w.g, w.dh16, BH, S, Spad, D, h_dtype, dtype, st)) != MLSTM_OK)
            return rc;
        const size_t vec = static_cast<size_t>(BH) * Spad * sizeof(float);
        const size_t mat = al(scan_gemm_bwd_matrix_bytes(BH, S, dtype));
        uint8_t* extra_base = static_cast<uint8_t*>(workspace) + w.bytes;
        ScanGemmBwdArgs a{};
        a.S = S; a.Spad = Spad; a.BH = BH; a.D = D;
        a.q = q; a.k = k; a.v = v; a.dh = need16 ? w.dh16 : dh;
        a.dq = dq; a.dk = dk; a.dv = dv;
        a.ga = w.ga; a.gaw = w.gaw; a.gB = w.gB; a.g = w.g; a.a_ref = w.a_ref; a.An_ref = w.An_ref;
        a.Wn = extra_base; a.dT = extra_base + mat;
        a.R = reinterpret_cast<float*>(extra_base + 2 * mat);
        a.dI = reinterpret_cast<float*>(extra_base + 2 * mat + al(vec * (D / 256)));
        a.dot_stride = static_cast<long long>(BH) * Spad;
        a.status = w.status; a.counters = w.status + 8 + 12;
        if ((rc = launch_scan_gemm_bwd(a, dtype, st)) != MLSTM_OK) return rc;
        return launch_df(f, a.dI, a.R, df, di, BH, S, Spad, dtype, st, D / 256, a.dot_stride);
    }
    const size_t extra = tf32_copy_bytes(BH, S, D, dtype, flags, 4);
    if (!workspace || workspace_bytes < w.bytes + extra || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    const int kind = pass_kind(S, D, dtype, flags, &rc);
    if (rc != MLSTM_OK) return rc;

    if ((rc = launch_gates_fwd(f, i, w.ga, w.gAn, w.a_ref, w.An_ref, nullptr, BH, S, Spad, dtype, st, nullptr, nullptr, nullptr, 0,
                               nullptr, w.gaw, w.status, STATUS_WORDS)) != MLSTM_OK)
        return rc;
    if ((rc = launch_bwd_prep(h, dh, b, m, w.gAn, w.gB, w.gBw, w.g, w.dh16, BH, S, Spad, D, h_dtype, dtype, st)) != MLSTM_OK)
        return rc;
    const void* dhp = need16 ? w.dh16 : dh;  // dh in the element type of q, k, v
    const void* orig_q = q;
    const void* orig_k = k;
    if (kind != KIND_SIMT && dtype == MLSTM_DT_F32) {  // converted copies of q, k, v, dh
        if (!extra) return MLSTM_E_WORKSPACE;
        const void* in[4] = {q, k, v, dhp};
        if ((rc = round_inputs(in, 4, static_cast<uint8_t*>(workspace) + w.bytes, BH, S, D, kind, st)) != MLSTM_OK) return rc;
        q = in[0]; k = in[1]; v = in[2]; dhp = in[3];
    }

    PassParams p{};
    p.S = S; p.Spad = Spad; p.BH = BH; p.D = D; p.status = w.status; p.sched = w.status + 8; p.sched_zeroed = 1;
    p.dot_part_stride = static_cast<long long>(BH) * Spad;
    // dQ = ((dH V^T + g_r) * decay) K
    p.X = dhp; p.Y = v; p.Z = k;
    p.row_rel = w.gB; p.row_ref = w.An_ref; p.row_g = w.g; p.col_rel = w.ga; p.col_w = w.gaw; p.col_ref = w.a_ref; p.col_g = nullptr;
    p.out = dq; p.dot_src = orig_q; p.dot_out = w.R;
    if ((rc = run_pass(kind, DQ, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    // dK = ((V dH^T + g_c) * decay)  Q
    p.X = v; p.Y = dhp; p.Z = q;
    p.row_rel = w.ga; p.row_ref = w.a_ref; p.row_g = nullptr; p.col_rel = w.gB; p.col_w = w.gBw; p.col_ref = w.An_ref; p.col_g = w.g;
    p.out = dk; p.dot_src = orig_k; p.dot_out = w.dI;
    if ((rc = run_pass(kind, DK, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    // dV = ((K Q^T) * decay / n) dH
    p.X = k; p.Y = q; p.Z = dhp;
    p.col_g = nullptr;
    p.out = dv; p.dot_src = nullptr; p.dot_out = nullptr;
    if ((rc = run_pass(kind, DV, p, dtype, dtype, st)) != MLSTM_OK) return rc;
    return launch_df(f, w.dI, w.R, df, di, BH, S, Spad, dtype, st, kind == KIND_SIMT ? 1 : TC_DOT_PARTS,
                     static_cast<long long>(BH) * Spad);
}

// Which of its three forms the scan entry uses.
//   TWO_PASS   head dimension above 256: gated S x S matrix once, then W V (scan_gemm.cu)
//   CHUNKWISE  sequence much longer than the head dimension: per-block states (C, n) with the stabiliser
//              known up front, inter-block carry, output from the carried state (chunk.cu; the mechanism of
//              mlstm_scan.py:74-137, 143-195, 200-278)
//   QUADRATIC  the parallel forward with the output gate in its epilogue
enum ScanRoute { SCAN_QUADRATIC = 0, SCAN_TWO_PASS = 1, SCAN_CHUNKWISE = 2 };
constexpr int SCAN_CHUNK = 256;

static int scan_route(int B, int NH, int S, int D, int dtype, int flags) {
    const bool math_ok = dtype != MLSTM_DT_F32 || (flags & MLSTM_F_ALLOW_TF32);
    if (flags & MLSTM_F_FORCE_SIMT) return SCAN_QUADRATIC;
    if (scan_gemm_supported(S, D, dtype) && math_ok) return SCAN_TWO_PASS;
    // the state form does 4 S D^2 flops per slice beside the blocks' own triangles, the quadratic form 2 S^2 D
    if (S > 2 * D && S > 2 * SCAN_CHUNK && mlstm_chunk_workspace(B, NH, S, D, dtype, SCAN_CHUNK) != 0) return SCAN_CHUNKWISE;
    return SCAN_QUADRATIC;
}

size_t mlstm_scan_fwd_workspace(int B, int NH, int S, int D, int dtype, int flags) {
    if (check_dims(B, NH, S, D) != MLSTM_OK) return 0;
    switch (scan_route(B, NH, S, D, dtype, flags)) {
        case SCAN_TWO_PASS:
            return carve_fwd(nullptr, B * NH, S, true).bytes + two_pass_extra_bytes(B * NH, S, dtype);
        case SCAN_CHUNKWISE: return mlstm_chunk_workspace(B, NH, S, D, dtype, SCAN_CHUNK);
        default: return carve_fwd(nullptr, B * NH, S, true).bytes + tf32_copy_bytes(B * NH, S, D, dtype, flags, 3);
    }
}

int mlstm_scan_fwd(const void* q, const void* k, const void* v, const void* f, const void* i, const void* o, void* h,
                   void* workspace, size_t workspace_bytes, int B, int NH, int S, int D, int dtype, int flags,
                   void* stream) {
    if (!q || !k || !v || !f || !i || !o || !h) return MLSTM_E_ARG;
    if (!dtype_ok(dtype)) return MLSTM_E_ARG;
    int rc = check_dims(B, NH, S, D);
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(h)) return MLSTM_E_ALIGN;
    const int BH = B * NH;
    const size_t need = mlstm_scan_fwd_workspace(B, NH, S, D, dtype, flags);
    if (!workspace || need == 0 || workspace_bytes < need || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int route = scan_route(B, NH, S, D, dtype, flags);
    if (route == SCAN_CHUNKWISE) {
        if ((rc = mlstm_chunk_prepare(k, v, f, i, nullptr, nullptr, workspace, workspace_bytes, B, NH, S, D, dtype, SCAN_CHUNK,
                                      stream)) != MLSTM_OK)
            return rc;
        return mlstm_chunk_apply(q, k, v, o, nullptr, nullptr, h, MLSTM_DT_F32, nullptr, nullptr, workspace, workspace_bytes,
                                 B, NH, S, D, dtype, SCAN_CHUNK, stream);
    }
    FwdWs w = carve_fwd(workspace, BH, S, true);
    if (route == SCAN_TWO_PASS)
        return two_pass_forward(q, k, v, f, i, o, static_cast<float*>(h), w.m, nullptr, w, static_cast<uint8_t*>(workspace) + w.bytes,
                                BH, S, D, dtype, st);
    if ((flags & MLSTM_F_FORCE_TC) && D > 256) return MLSTM_E_UNSUPPORTED;
    const size_t extra = tf32_copy_bytes(BH, S, D, dtype, flags, 3);
    void* tf32buf = extra ? static_cast<uint8_t*>(workspace) + w.bytes : nullptr;
    return forward_impl(q, k, v, f, i, o, h, w.m, w.b, w, BH, S, D, dtype, MLSTM_DT_F32, flags, st, tf32buf);
}

int mlstm_ogate_fwd(const void* h_inner, const void* o, void* h, long long n, int h_dtype, int o_dtype, void* stream) {
    if (!h_inner || !o || !h || n <= 0) return MLSTM_E_ARG;
    if (!dtype_ok(h_dtype) || !dtype_ok(o_dtype)) return MLSTM_E_ARG;
    return launch_ogate_fwd(h_inner, o, h, n, h_dtype, o_dtype, static_cast<cudaStream_t>(stream));
}

int mlstm_ogate_bwd(const void* dh, const void* h_inner, const void* o, void* dh_inner, void* d_o, long long n, int h_dtype,
                    int o_dtype, void* stream) {
    if (!dh || !h_inner || !o || !dh_inner || !d_o || n <= 0) return MLSTM_E_ARG;
    if (!dtype_ok(h_dtype) || !dtype_ok(o_dtype)) return MLSTM_E_ARG;
    return launch_ogate_bwd(dh, h_inner, o, dh_inner, d_o, n, h_dtype, o_dtype, static_cast<cudaStream_t>(stream));
}

size_t mlstm_forward_f16_workspace(unsigned S, unsigned D) {
    if (check_dims(1, 1, static_cast<int>(S), static_cast<int>(D)) != MLSTM_OK) return 0;
    return carve_fwd(nullptr, 1, static_cast<int>(S), true).bytes;
}

int mlstm_forward_f16(const void* Q, const void* K, const void* V, const void* F, const void* I, void* H, unsigned S,
                      unsigned D, void* workspace, size_t workspace_bytes, void* stream) {
    if (!Q || !K || !V || !F || !I || !H) return MLSTM_E_ARG;
    if (S > 0x7fffffffu || D > 0x7fffffffu) return MLSTM_E_ARG;
    int rc = check_dims(1, 1, static_cast<int>(S), static_cast<int>(D));
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(H)) return MLSTM_E_ALIGN;
    FwdWs w = carve_fwd(workspace, 1, static_cast<int>(S), true);
    if (!workspace || workspace_bytes < w.bytes || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    return forward_impl(Q, K, V, F, I, nullptr, H, w.m, w.b, w, 1, static_cast<int>(S), static_cast<int>(D), MLSTM_DT_F16,
                        MLSTM_DT_F16, 0, static_cast<cudaStream_t>(stream));
}

// Single-head fp16 backward of the C++ driver: the forward is run first for h, m and b (the reference's
// launches take M and B from a host computation and have no h; the row dots delta = dh . h used here need it),
// then the three backward passes and the dF scan.  Workspace: forward scratch | h [S, D] half | backward scratch.
static size_t bwd16_h_offset(int S) { return carve_fwd(nullptr, 1, S, true).bytes; }
static size_t bwd16_bwd_offset(int S, int D) { return bwd16_h_offset(S) + al(static_cast<size_t>(S) * D * 2); }

size_t mlstm_backward_f16_workspace(unsigned S, unsigned D) {
    if (S > 0x7fffffffu || D > 0x7fffffffu) return 0;
    if (check_dims(1, 1, static_cast<int>(S), static_cast<int>(D)) != MLSTM_OK) return 0;
    return bwd16_bwd_offset(static_cast<int>(S), static_cast<int>(D)) +
           mlstm_mm_bwd_workspace(1, 1, static_cast<int>(S), static_cast<int>(D), MLSTM_DT_F16, MLSTM_DT_F16, 0);
}

int mlstm_backward_f16(const void* dH, const void* Q, const void* K, const void* V, const void* F, const void* I, void* dQ,
                       void* dK, void* dV, void* dF, void* dI, unsigned S, unsigned D, void* workspace,
                       size_t workspace_bytes, void* stream) {
    if (!dH || !Q || !K || !V || !F || !I || !dQ || !dK || !dV || !dF || !dI) return MLSTM_E_ARG;
    if (S > 0x7fffffffu || D > 0x7fffffffu) return MLSTM_E_ARG;
    const int s = static_cast<int>(S), d = static_cast<int>(D);
    int rc = check_dims(1, 1, s, d);
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(dH) || !aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(dQ) || !aligned16(dK) || !aligned16(dV))
        return MLSTM_E_ALIGN;
    const size_t need = mlstm_backward_f16_workspace(S, D);
    if (!workspace || need == 0 || workspace_bytes < need || !aligned16(workspace)) return MLSTM_E_WORKSPACE;
    uint8_t* base = static_cast<uint8_t*>(workspace);
    FwdWs w = carve_fwd(base, 1, s, true);
    void* h = base + bwd16_h_offset(s);
    rc = forward_impl(Q, K, V, F, I, nullptr, h, w.m, w.b, w, 1, s, d, MLSTM_DT_F16, MLSTM_DT_F16, 0,
                      static_cast<cudaStream_t>(stream));
    if (rc != MLSTM_OK) return rc;
    const size_t off = bwd16_bwd_offset(s, d);
    return mlstm_mm_bwd(dH, Q, K, V, F, I, h, w.m, w.b, dQ, dK, dV, dF, dI, base + off, workspace_bytes - off, 1, 1, s, d,
                        MLSTM_DT_F16, MLSTM_DT_F16, 0, stream);
}

// ------------------------------------------------------------------------------------------------
// Single-head fp16 forward for callers that have no way to hand over scratch memory.
//
// The C++ driver's launch (Q, K, V, F, I, H, S) has no workspace argument, and some of its callers
// cannot create one: code on a latency-critical path, where cudaMalloc and cudaFree serialise the
// whole device, and embedders that were given a fixed memory budget and no allocator.  For them the
// scratch of the forward (status word, the three gate vectors with their block references, m and b)
// lives in one array in the library's device image.  It costs MLSTM_STATIC_SCRATCH_BYTES on every
// GPU that loads the library, for as long as the process lives, hence the modest length limit.
//
// In host code the array's name is only a handle of the host-side shadow; its device address comes
// from cudaGetSymbolAddress, asked once per device with that device current, on the first call
// there.  That first call must therefore not happen inside a stream capture.  All calls on one
// device share the array: the status word is cleared at the start of each call, everything else is
// rewritten before it is read, and two calls whose kernels overlap on the GPU (different streams,
// no dependency) corrupt each other.
constexpr unsigned STATIC_MAX_S = MLSTM_STATIC_MAX_S;
static_assert(fwd_layout(1, STATIC_MAX_S, true).bytes == MLSTM_STATIC_SCRATCH_BYTES,
              "the header's figure must be the forward scratch of one head at MLSTM_STATIC_MAX_S");
static __device__ __align__(256) unsigned char g_static_scratch[MLSTM_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out) {
    constexpr int MAX_DEVICES = 64;
    static std::mutex mu;
    static void* addr[MAX_DEVICES] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return MLSTM_E_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return MLSTM_E_CUDA;
        }
        addr[dev] = p;
    }
    *out = addr[dev];
    return MLSTM_OK;
}

int mlstm_forward_f16_static(const void* Q, const void* K, const void* V, const void* F, const void* I, void* H,
                             unsigned S, unsigned D, void* stream) {
    if (!Q || !K || !V || !F || !I || !H) return MLSTM_E_ARG;
    if (S == 0 || D == 0 || D > 0x7fffffffu) return MLSTM_E_ARG;
    if (S > STATIC_MAX_S) return MLSTM_E_STATIC_LIMIT;
    int rc = check_dims(1, 1, static_cast<int>(S), static_cast<int>(D));
    if (rc != MLSTM_OK) return rc;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(H)) return MLSTM_E_ALIGN;
    void* scratch = nullptr;
    if ((rc = static_scratch_address(&scratch)) != MLSTM_OK) return rc;
    FwdWs w = carve_fwd(scratch, 1, static_cast<int>(S), true);
    if (w.bytes > MLSTM_STATIC_SCRATCH_BYTES) return MLSTM_E_STATIC_LIMIT;
    return forward_impl(Q, K, V, F, I, nullptr, H, w.m, w.b, w, 1, static_cast<int>(S), static_cast<int>(D), MLSTM_DT_F16,
                        MLSTM_DT_F16, 0, static_cast<cudaStream_t>(stream));
}

int mlstm_forward_f16_static_status(int* host_status, void* stream) {
    if (!host_status) return MLSTM_E_ARG;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != MLSTM_OK) return rc;
    return mlstm_read_status(scratch, host_status, stream);
}

int mlstm_read_status(const void* workspace, int* host_status, void* stream) {
    if (!workspace || !host_status) return MLSTM_E_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaStreamSynchronize(st) != cudaSuccess) return MLSTM_E_CUDA;
    if (cudaMemcpy(host_status, workspace, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MLSTM_E_CUDA;
    return *host_status == 0 ? MLSTM_OK : MLSTM_E_TIMEOUT;
}

}  // extern "C"
