// C entry points of the fused flash-SDPA tile tasks: argument checks and the
// choice between the tcgen05 kernels and the generic CUDA kernels.  Both are
// device code; there is no host fallback.
#include "flash.cuh"

using namespace nb200;

static int check_common(int64_t seq, int64_t head, int64_t batch)
{
    if(seq < 0 || head < 0 || batch < 0) return NNTILE_B200_E_BADARG;
    if(head > 256 || seq > (int64_t)1 << 24) return NNTILE_B200_E_SHAPE;
    return NNTILE_B200_OK;
}

#ifndef NB200_FP16
extern "C" int nntile_b200_flash_sdpa_fwd_path(int64_t seq, int64_t head, int64_t batch)
{
    if(check_common(seq, head, batch) != NNTILE_B200_OK) return 0;
    return flash_fwd_sm100_supports(seq, head, batch) ? 2 : 1;
}

extern "C" int nntile_b200_flash_sdpa_bwd_path(int64_t seq, int64_t head, int64_t batch)
{
    if(check_common(seq, head, batch) != NNTILE_B200_OK || head < 2) return 0;
    return flash_bwd_sm100_supports(seq, head, batch) ? 2 : 1;
}

#endif // NB200_FP16

namespace nb200 {
inline namespace NB200_ELEM_NS {

int flash_fwd_task(cudaStream_t stream, Index seq, Index head, Index batch, const void *K,
        const void *Q, const void *mask, const void *V, void *scratch_A, float *lse, void *A,
        const FwdAux *fwd_aux)
{
    int st = check_common(seq, head, batch);
    if(st != NNTILE_B200_OK) return st;
    if(seq == 0 || head == 0 || batch == 0) return NNTILE_B200_OK;
    if(!K || !Q || !mask || !V || !lse || !A) return NNTILE_B200_E_BADARG;
    if(flash_fwd_sm100_supports(seq, head, batch))
    {
        if(!fwd_aux && !scratch_A) return NNTILE_B200_E_BADARG;
        if(!aligned16(K) || !aligned16(Q) || !aligned16(V) || !aligned16(A)
                || !aligned16(mask) || (!fwd_aux && !aligned16(scratch_A)))
        {
            return NNTILE_B200_E_ALIGN;
        }
        FwdAux aux;
        if(fwd_aux)
        {
            aux = *fwd_aux;
        }
        else
        {
            // status word + class table at the start of the task's scratch buffer
            const size_t nblk = (size_t)(seq/128);
            if((size_t)seq*head*batch*sizeof(elem_t) < CLS_OFFSET + nblk*nblk)
            {
                return NNTILE_B200_E_SCRATCH;
            }
            uint8_t *sc = static_cast<uint8_t *>(scratch_A);
            aux.status = reinterpret_cast<uint32_t *>(sc);
            aux.cls = sc + CLS_OFFSET;
            aux.classify = true;
        }
        return flash_fwd_sm100(stream, seq, head, batch, (const elem_t *)K, (const elem_t *)Q,
                (const elem_t *)mask, (const elem_t *)V, lse, (elem_t *)A, aux, 1, batch);
    }
    return flash_fwd_generic(stream, seq, head, batch, (const elem_t *)K, (const elem_t *)Q,
            (const elem_t *)mask, (const elem_t *)V, lse, (elem_t *)A);
}

int flash_bwd_task(cudaStream_t stream, Index seq, Index head, Index batch, const void *K,
        const void *Q, const void *V, const void *A, const void *dA, const void *mask,
        const float *lse, void *scratch_dK, void *scratch_dQ, void *scratch_dV, void *dK,
        void *dQ, void *dV, const BwdAux *bwd_aux)
{
    int st = check_common(seq, head, batch);
    if(st != NNTILE_B200_OK) return st;
    if(seq == 0 || head == 0 || batch == 0) return NNTILE_B200_OK;
    if(!K || !Q || !V || !A || !dA || !mask || !lse || !dK || !dQ || !dV)
    {
        return NNTILE_B200_E_BADARG;
    }
    const bool fast = flash_bwd_sm100_supports(seq, head, batch);
    if(!(bwd_aux && fast))
    {
        if(!scratch_dK || !scratch_dQ || !scratch_dV) return NNTILE_B200_E_BADARG;
        // delta (seq*batch floats) lives in scratch_dV: needs head >= 2
        if(head < 2) return NNTILE_B200_E_SHAPE;
        if(!aligned16(scratch_dV) || !aligned16(scratch_dQ) || !aligned16(scratch_dK))
        {
            return NNTILE_B200_E_ALIGN;
        }
    }
    if(fast)
    {
        if(!aligned16(K) || !aligned16(Q) || !aligned16(V) || !aligned16(A)
                || !aligned16(dA) || !aligned16(mask) || !aligned16(dK)
                || !aligned16(dQ) || !aligned16(dV))
        {
            return NNTILE_B200_E_ALIGN;
        }
        const BwdAux aux = bwd_aux ? *bwd_aux
                : bwd_aux_from_scratch(seq, batch, scratch_dK, scratch_dQ, scratch_dV);
        return flash_bwd_sm100(stream, seq, head, batch, (const elem_t *)K, (const elem_t *)Q,
                (const elem_t *)V, (const elem_t *)A, (const elem_t *)dA, (const elem_t *)mask, lse, aux,
                (elem_t *)dK, (elem_t *)dQ, (elem_t *)dV, 1, batch);
    }
    return flash_bwd_generic(stream, seq, head, batch, (const elem_t *)K, (const elem_t *)Q,
            (const elem_t *)V, (const elem_t *)A, (const elem_t *)dA, (const elem_t *)mask, lse,
            (float *)scratch_dV, (elem_t *)dK, (elem_t *)dQ, (elem_t *)dV);
}

} // inline namespace
} // namespace nb200

extern "C" int NB200_SFX(nntile_b200_flash_sdpa_fwd)(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q, const void *mask,
        float *scratch_lse, const void *V, void *scratch_A, float *lse, void *A)
{
    (void)scratch_lse;
    return flash_fwd_task(as_stream(stream), seq, head, batch, K, Q, mask, V, scratch_A, lse, A,
            nullptr);
}

extern "C" int NB200_SFX(nntile_b200_flash_sdpa_bwd)(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q, const void *V,
        const void *A, const void *dA, const void *mask, const float *lse,
        void *scratch_dK, void *scratch_dQ, void *scratch_dV, void *dK, void *dQ, void *dV)
{
    return flash_bwd_task(as_stream(stream), seq, head, batch, K, Q, V, A, dA, mask, lse,
            scratch_dK, scratch_dQ, scratch_dV, dK, dQ, dV, nullptr);
}

#ifndef NB200_FP16
// The status word of the fused kernels sits in the first four bytes of the scratch
// buffer that carries a task's bookkeeping; this reads it back after the stream
// has drained.
extern "C" int nntile_b200_flash_sdpa_read_status(nntile_b200_stream_t stream,
        const void *scratch, unsigned int *code)
{
    if(!scratch || !code) return NNTILE_B200_E_BADARG;
    uint32_t word = 0;
    if(cudaMemcpyAsync(&word, scratch, sizeof(word), cudaMemcpyDeviceToHost, as_stream(stream))
            != cudaSuccess || cudaStreamSynchronize(as_stream(stream)) != cudaSuccess)
    {
        return NNTILE_B200_E_LAUNCH;
    }
    *code = word;
    return NNTILE_B200_OK;
}

#endif // NB200_FP16

// ------------------------------------------------------------ grouped-query form
// Q, A, dA, dQ: [head, seq, batch, group, kv_heads]; K, V, dK, dV: [head, seq, batch,
// kv_heads] (not replicated over the group).  tcgen05 kernels only.
static int check_gqa(int64_t seq, int64_t head, int64_t batch, int64_t group, int64_t kv_heads)
{
    if(seq < 0 || head < 0 || batch < 0 || group < 0 || kv_heads < 0) return NNTILE_B200_E_BADARG;
    return NNTILE_B200_OK;
}

#ifndef NB200_FP16
extern "C" size_t nntile_b200_flash_sdpa_gqa_scratch_bytes(int64_t seq, int64_t head,
        int64_t batch, int64_t group, int64_t kv_heads)
{
    if(check_gqa(seq, head, batch, group, kv_heads) != NNTILE_B200_OK) return 0;
    // status word + class table + delta + lse*log2e in a region the size of one
    // elem_t tensor, then the fp32 dQ accumulator
    return (size_t)seq*head*batch*group*kv_heads*6;
}

#endif // NB200_FP16

extern "C" int NB200_SFX(nntile_b200_flash_sdpa_fwd_gqa)(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *mask, const void *V, float *lse, void *A, void *scratch,
        size_t scratch_bytes)
{
    int st = check_gqa(seq, head, batch, group, kv_heads);
    if(st != NNTILE_B200_OK) return st;
    const int64_t slices = batch*group*kv_heads;
    if(seq == 0 || head == 0 || slices == 0) return NNTILE_B200_OK;
    if(!K || !Q || !mask || !V || !lse || !A || !scratch) return NNTILE_B200_E_BADARG;
    if(!flash_fwd_sm100_supports(seq, head, slices)) return NNTILE_B200_E_SHAPE;
    if(!aligned16(K) || !aligned16(Q) || !aligned16(V) || !aligned16(A) || !aligned16(mask)
            || !aligned16(scratch))
    {
        return NNTILE_B200_E_ALIGN;
    }
    const size_t nblk = (size_t)(seq/128);
    if(scratch_bytes < CLS_OFFSET + nblk*nblk) return NNTILE_B200_E_SCRATCH;
    uint8_t *sc = static_cast<uint8_t *>(scratch);
    const FwdAux aux = {reinterpret_cast<uint32_t *>(sc), sc + CLS_OFFSET, true};
    return flash_fwd_sm100(as_stream(stream), seq, head, slices, (const elem_t *)K,
            (const elem_t *)Q, (const elem_t *)mask, (const elem_t *)V, lse, (elem_t *)A, aux, group,
            batch);
}

extern "C" int NB200_SFX(nntile_b200_flash_sdpa_bwd_gqa)(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *V, const void *A, const void *dA, const void *mask,
        const float *lse, void *dK, void *dQ, void *dV, void *scratch, size_t scratch_bytes)
{
    int st = check_gqa(seq, head, batch, group, kv_heads);
    if(st != NNTILE_B200_OK) return st;
    const int64_t slices = batch*group*kv_heads;
    if(seq == 0 || head == 0 || slices == 0) return NNTILE_B200_OK;
    if(!K || !Q || !V || !A || !dA || !mask || !lse || !dK || !dQ || !dV || !scratch)
    {
        return NNTILE_B200_E_BADARG;
    }
    if(!flash_bwd_sm100_supports(seq, head, slices)) return NNTILE_B200_E_SHAPE;
    if(scratch_bytes < nntile_b200_flash_sdpa_gqa_scratch_bytes(seq, head, batch, group, kv_heads))
    {
        return NNTILE_B200_E_SCRATCH;
    }
    if(!aligned16(K) || !aligned16(Q) || !aligned16(V) || !aligned16(A) || !aligned16(dA)
            || !aligned16(mask) || !aligned16(dK) || !aligned16(dQ) || !aligned16(dV)
            || !aligned16(scratch))
    {
        return NNTILE_B200_E_ALIGN;
    }
    const size_t part = (size_t)seq*head*slices*2;        // one elem_t tensor of Q's shape
    uint8_t *sc = static_cast<uint8_t *>(scratch);
    const BwdAux aux = bwd_aux_from_scratch(seq, slices, sc + 2*part, sc + part, sc);
    return flash_bwd_sm100(as_stream(stream), seq, head, slices, (const elem_t *)K,
            (const elem_t *)Q, (const elem_t *)V, (const elem_t *)A, (const elem_t *)dA,
            (const elem_t *)mask, lse, aux, (elem_t *)dK, (elem_t *)dQ, (elem_t *)dV, group, batch);
}
