// C-ABI entry points of the chunk kernels: argument checks, then the launcher of the tensor-core kernel.
#include "host.h"

using namespace mkda;

extern "C" int mkda_intra_fwd(const MkdaIntraFwd* p, void* stream) {
    if (!p || !p->q || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->Aqk || !p->nw || !p->u || !p->kbar || !p->qs || !p->gl)
        return set_error(MKDA_ERR_ARG, "intra_fwd: null argument");
    if (any_misaligned(p->q, p->k, p->v, p->g_c, p->A, p->Aqk, p->nw, p->u, p->kbar, p->qs, p->gl))
        return set_error(MKDA_ERR_ARG, "intra_fwd: tensors must be 16-byte aligned");
    if (p->L.HK <= 0 || p->L.HV % p->L.HK) return set_error(MKDA_ERR_ARG, "intra_fwd: HV must be a multiple of HK");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_intra_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_recur_fwd(const MkdaRecurFwd* p, void* stream) {
    if (!p || !p->nw || !p->u || !p->kbar || !p->gl) return set_error(MKDA_ERR_ARG, "recur_fwd: null argument");
    if (any_misaligned(p->nw, p->u, p->kbar, p->gl, p->h, p->Vd)) return set_error(MKDA_ERR_ARG, "recur_fwd: tensors must be 16-byte aligned");
    if (p->want_transition && !p->mt) return set_error(MKDA_ERR_ARG, "recur_fwd: want_transition needs mt");
    if (p->L.NS == 0) return MKDA_OK;
    return launch_recur_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_out_fwd(const MkdaOutFwd* p, void* stream) {
    if (!p || !p->qs || !p->Aqk || !p->Vd || !p->h || !p->out) return set_error(MKDA_ERR_ARG, "out_fwd: null argument");
    if (any_misaligned(p->qs, p->Aqk, p->Vd, p->h, p->out, p->o_raw, p->gate, p->norm_w)) return set_error(MKDA_ERR_ARG, "out_fwd: tensors must be 16-byte aligned");
    if (p->has_norm && !p->gate) return set_error(MKDA_ERR_ARG, "out_fwd: the gated norm needs a gate tensor");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_out_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_bwd_dh(const MkdaBwdDh* p, void* stream) {
    if (!p || (!p->d_o && !p->dO_in_t) || !p->kbar || !p->qs || !p->gl || !p->Aqk || !p->nw)
        return set_error(MKDA_ERR_ARG, "bwd_dh: null argument");
    if (any_misaligned(p->d_o, p->dO_in_t, p->kbar, p->qs, p->gl, p->Aqk, p->nw, p->dh, p->dVd_t, p->dO_t))
        return set_error(MKDA_ERR_ARG, "bwd_dh: tensors must be 16-byte aligned");
    if (p->L.NS == 0) return MKDA_OK;
    return launch_bwd_dh_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_bwd_chunk(const MkdaBwdChunk* p, void* stream) {
    if (!p || !p->q || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->h || !p->dh || !p->Vd || !p->dO_t || !p->dVd_t ||
        !p->dq_v || !p->dk_v || !p->dgp || !p->dbeta || !p->dv)
        return set_error(MKDA_ERR_ARG, "bwd_chunk: null argument");
    if (any_misaligned(p->q, p->k, p->v, p->g_c, p->A, p->h, p->dh, p->Vd, p->dO_t, p->dVd_t, p->dq_v, p->dk_v, p->dgp, p->dv))
        return set_error(MKDA_ERR_ARG, "bwd_chunk: tensors must be 16-byte aligned");
    if (p->beta_sigmoid && !p->beta_raw) return set_error(MKDA_ERR_ARG, "bwd_chunk: sigmoid beta needs the raw input");
    if (p->L.HK <= 0 || p->L.HV % p->L.HK) return set_error(MKDA_ERR_ARG, "bwd_chunk: HV must be a multiple of HK");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_bwd_chunk_tc(p, (cudaStream_t)stream);
}
