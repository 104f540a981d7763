// TEST INFRASTRUCTURE ONLY.  The instruction sequence of the reference's multi-latent-attention demo
// (demos/cpu/mla_attention_demo/mla_attention_demo.cpp:326-376) with fp16 matrix operands, run on the reference's own
// CPU simulation (compiled against its headers where they lie, see Makefile).  It is the oracle for the same sequence
// issued on the B200 PTO surface (pto_isa_b200/csrc/pto_programs/programs.cu: ProgMlaHead); nothing in the product
// links or calls it.  Every accumulator goes Acc -> Vec fp32 (TMOV) -> fp16 (TCVT, CAST_RINT) -> Left / Right (TMOV).
#include <pto/pto-inst.hpp>

#include <cstdint>
#include <memory>

using namespace pto;

namespace {

template <int S, int D, int R>
void MlaHead(float *out, const half *q, const half *k, const half *v, const half *wq, const half *wk, const half *wv,
             const half *wo, float scale)
{
    using GSD = GlobalTensor<half, Shape<1, 1, 1, S, D>, pto::Stride<S * D, S * D, S * D, D, 1>>;
    using GDR = GlobalTensor<half, Shape<1, 1, 1, D, R>, pto::Stride<D * R, D * R, D * R, R, 1>>;
    using GRD = GlobalTensor<half, Shape<1, 1, 1, R, D>, pto::Stride<R * D, R * D, R * D, D, 1>>;
    using GO = GlobalTensor<float, Shape<1, 1, 1, S, D>, pto::Stride<S * D, S * D, S * D, D, 1>>;
    using SDh = Tile<TileType::Vec, half, S, D, BLayout::RowMajor, S, D, SLayout::NoneBox>;
    using DRh = Tile<TileType::Vec, half, D, R, BLayout::RowMajor, D, R, SLayout::NoneBox>;
    using RDh = Tile<TileType::Vec, half, R, D, BLayout::RowMajor, R, D, SLayout::NoneBox>;
    using SRh = Tile<TileType::Vec, half, S, R, BLayout::RowMajor, S, R, SLayout::NoneBox>;
    using RSh = Tile<TileType::Vec, half, R, S, BLayout::RowMajor, R, S, SLayout::NoneBox>;
    using SRf = Tile<TileType::Vec, float, S, R, BLayout::RowMajor, S, R, SLayout::NoneBox>;
    using SSf = Tile<TileType::Vec, float, S, S, BLayout::RowMajor, S, S, SLayout::NoneBox>;
    using SSh = Tile<TileType::Vec, half, S, S, BLayout::RowMajor, S, S, SLayout::NoneBox>;
    using SDf = Tile<TileType::Vec, float, S, D, BLayout::RowMajor, S, D, SLayout::NoneBox>;
    using RowRed = Tile<TileType::Vec, float, S, 1, BLayout::ColMajor, S, 1, SLayout::NoneBox>;

    auto qv = std::make_unique<SDh>(), kv = std::make_unique<SDh>(), vv = std::make_unique<SDh>();
    auto wqv = std::make_unique<DRh>(), wkv = std::make_unique<DRh>(), wvv = std::make_unique<DRh>();
    auto wov = std::make_unique<RDh>();
    auto qlat = std::make_unique<SRh>(), klat = std::make_unique<SRh>(), vlat = std::make_unique<SRh>();
    auto ctx16 = std::make_unique<SRh>();
    auto klat_t = std::make_unique<RSh>();
    auto tmp32 = std::make_unique<SRf>();
    auto scores = std::make_unique<SSf>();
    auto probs = std::make_unique<SSh>();
    auto mx = std::make_unique<RowRed>(), sm = std::make_unique<RowRed>();
    auto l_sd = std::make_unique<TileLeft<half, S, D, S, D>>();
    auto l_sr = std::make_unique<TileLeft<half, S, R, S, R>>();
    auto l_ss = std::make_unique<TileLeft<half, S, S, S, S>>();
    auto r_wq = std::make_unique<TileRight<half, D, R, D, R>>(), r_wk = std::make_unique<TileRight<half, D, R, D, R>>(),
         r_wv = std::make_unique<TileRight<half, D, R, D, R>>();
    auto r_wo = std::make_unique<TileRight<half, R, D, R, D>>();
    auto r_klat_t = std::make_unique<TileRight<half, R, S, R, S>>();
    auto r_vlat = std::make_unique<TileRight<half, S, R, S, R>>();
    auto acc_sr = std::make_unique<TileAcc<float, S, R, S, R>>();
    auto acc_ss = std::make_unique<TileAcc<float, S, S, S, S>>();
    auto acc_sd = std::make_unique<TileAcc<float, S, D, S, D>>();
    auto out_v = std::make_unique<SDf>();

    GSD gq(const_cast<half *>(q)), gk(const_cast<half *>(k)), gv(const_cast<half *>(v));
    GDR gwq(const_cast<half *>(wq)), gwk(const_cast<half *>(wk)), gwv(const_cast<half *>(wv));
    GRD gwo(const_cast<half *>(wo));
    GO go(out);
    TLOAD(*qv, gq);
    TLOAD(*kv, gk);
    TLOAD(*vv, gv);
    TLOAD(*wqv, gwq);
    TLOAD(*wkv, gwk);
    TLOAD(*wvv, gwv);
    TLOAD(*wov, gwo);
    TMOV(*r_wq, *wqv);
    TMOV(*r_wk, *wkv);
    TMOV(*r_wv, *wvv);
    TMOV(*r_wo, *wov);

    auto project = [&](SDh &x, TileRight<half, D, R, D, R> &w, SRh &dst) {
        TMOV(*l_sd, x);
        TMATMUL(*acc_sr, *l_sd, w);
        TMOV(*tmp32, *acc_sr);
        TCVT(dst, *tmp32, RoundMode::CAST_RINT);
    };
    project(*qv, *r_wq, *qlat);
    project(*kv, *r_wk, *klat);
    project(*vv, *r_wv, *vlat);

    TTRANS(*klat_t, *klat, *klat);
    TMOV(*r_klat_t, *klat_t);
    TMOV(*r_vlat, *vlat);
    TMOV(*l_sr, *qlat);
    TMATMUL(*acc_ss, *l_sr, *r_klat_t);
    TMOV(*scores, *acc_ss);
    TMULS(*scores, *scores, scale);

    TROWMAX(*mx, *scores, *scores);
    TROWEXPANDSUB(*scores, *scores, *mx);
    TEXP(*scores, *scores);
    TROWSUM(*sm, *scores, *scores);
    TROWEXPANDDIV(*scores, *scores, *sm);
    TCVT(*probs, *scores, RoundMode::CAST_RINT);

    TMOV(*l_ss, *probs);
    TMATMUL(*acc_sr, *l_ss, *r_vlat);
    TMOV(*tmp32, *acc_sr);
    TCVT(*ctx16, *tmp32, RoundMode::CAST_RINT);
    TMOV(*l_sr, *ctx16);
    TMATMUL(*acc_sd, *l_sr, *r_wo);
    TMOV(*out_v, *acc_sd);
    TSTORE(go, *out_v);
}

} // namespace

extern "C" int pto_ref_mla_head_f16_128x64x64(const uint16_t *q, const uint16_t *k, const uint16_t *v, const uint16_t *wq,
                                              const uint16_t *wk, const uint16_t *wv, const uint16_t *wo, float *out,
                                              float scale)
{
    auto h = [](const uint16_t *p) { return reinterpret_cast<const half *>(p); };
    MlaHead<128, 64, 64>(out, h(q), h(k), h(v), h(wq), h(wk), h(wv), h(wo), scale);
    return 0;
}
