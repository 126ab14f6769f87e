// C-ABI entry points of the chunk kernels: argument checks, then the launcher of the tensor-core kernel.
#include "host.h"

using namespace mkda;

extern "C" int mkda_intra_fwd(const MkdaIntraFwd* p, void* stream) {
    if (!p || !p->q || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->Aqk || !p->nw || !p->u || !p->kbar || !p->qs || !p->gl)
        return set_error(MKDA_ERR_ARG, "intra_fwd: null argument");
    if (p->L.HK <= 0 || p->L.HV % p->L.HK) return set_error(MKDA_ERR_ARG, "intra_fwd: HV must be a multiple of HK");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_intra_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_recur_fwd(const MkdaRecurFwd* p, void* stream) {
    if (!p || !p->nw || !p->u || !p->kbar || !p->gl) return set_error(MKDA_ERR_ARG, "recur_fwd: null argument");
    if (p->want_transition && !p->mt) return set_error(MKDA_ERR_ARG, "recur_fwd: want_transition needs mt");
    if (p->L.NS == 0) return MKDA_OK;
    return launch_recur_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_out_fwd(const MkdaOutFwd* p, void* stream) {
    if (!p || !p->qs || !p->Aqk || !p->Vd || !p->h || !p->out) return set_error(MKDA_ERR_ARG, "out_fwd: null argument");
    if (p->has_norm && !p->gate) return set_error(MKDA_ERR_ARG, "out_fwd: the gated norm needs a gate tensor");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_out_fwd_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_bwd_dh(const MkdaBwdDh* p, void* stream) {
    if (!p || !p->d_o || !p->kbar || !p->qs || !p->gl || !p->Aqk || !p->nw || !p->dh || !p->dVd)
        return set_error(MKDA_ERR_ARG, "bwd_dh: null argument");
    if (p->L.NS == 0) return MKDA_OK;
    return launch_bwd_dh_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_bwd_wy(const MkdaBwdWy* p, void* stream) {
    if (!p || !p->k || !p->v || !p->g_c || !p->beta || !p->A || !p->h || !p->d_o || !p->dVd || !p->Vd || !p->dX ||
        !p->dbeta_w || !p->dAqk || !p->dL)
        return set_error(MKDA_ERR_ARG, "bwd_wy: null argument");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_bwd_wy_tc(p, (cudaStream_t)stream);
}

extern "C" int mkda_bwd_tail(const MkdaBwdTail* p, void* stream) {
    if (!p || !p->q || !p->k || !p->g_c || !p->beta || !p->d_o || !p->dX || !p->Vd || !p->h || !p->dh || !p->dAqk || !p->dL ||
        !p->dbeta_w || !p->dq_v || !p->dk_v || !p->dgp || !p->dbeta)
        return set_error(MKDA_ERR_ARG, "bwd_tail: null argument");
    if (p->beta_sigmoid && !p->beta_raw) return set_error(MKDA_ERR_ARG, "bwd_tail: sigmoid beta needs the raw input");
    if (p->L.HK <= 0 || p->L.HV % p->L.HK) return set_error(MKDA_ERR_ARG, "bwd_tail: HV must be a multiple of HK");
    if (p->L.NC == 0) return MKDA_OK;
    return launch_bwd_tail_tc(p, (cudaStream_t)stream);
}
