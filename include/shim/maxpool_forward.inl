/*
 * Body fragment for MaxPoolLayer<Device::CUDA>::forward(const V& input), replacing the maxPoolForwardGpu call of
 * include/cuda/MaxPoolLayer.h:39-41.  Three cases, told apart by the plan:
 *   - the pool was folded into the preceding convolution's epilogue, or it is a later pool of an SPP block: its output
 *     is already written, nothing runs;
 *   - it is the first pool of an SPP block (yolov7.yml: 5 / 9 / 13 over one tensor, joined by routes): one pxe_spp
 *     call reads the common input once and writes every pool of the block where the plan wants it;
 *   - otherwise one pxe_maxpool per planned destination (its own tensor, or a channel slot of a route's buffer).
 *
 * Uses the reference's members output_, indexes_, batch(), channels(), height(), width(), outputs(), outHeight(),
 * outWidth(), kernel_, stride_, padding_, index(), model(), training(); added by the integration: model().pxePlan(),
 * model().layerAt(i) with pxeOutput() / outputs() / outHeight() / outWidth() / outChannels() and, on the pools of an
 * SPP block, pxeKernel().
 */
{
    const pxe_step* st = this->model().pxePlan().step(this->index());
    const long long plane = (long long)this->outHeight() * this->outWidth();
    if (st == nullptr || (st->op == PXE_STEP_MAXPOOL && st->layer == this->index())) {
        const int n = st != nullptr ? st->n_dests : 1;
        for (int k = 0; k < n; ++k) {
            pxe_shim::Slot s{this->output_.data(), this->outputs()};
            if (st != nullptr) {
                const pxe_dest& pd = st->dests[k];
                auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : this->index());
                s = pxe_shim::resolve(pd, this->output_.data(), this->outputs(), route.pxeOutput(), route.outputs(), plane);
            }
            PXE_CHECK(pxe_maxpool(nullptr, input.data(), 0, s.ptr, s.batch_stride,
                                  (k == 0 && this->training()) ? indexes_.data() : nullptr, this->batch(), this->channels(),
                                  this->height(), this->width(), kernel_, stride_, padding_));
        }
    } else if (st->op == PXE_STEP_SPP && st->layer == this->index()) {
        int kernels[PXE_PLAN_MAX_SPP];
        float* ys[PXE_PLAN_MAX_SPP];
        long long strides[PXE_PLAN_MAX_SPP];
        for (int g = 0; g < st->n_spp; ++g) {
            auto& pool = this->model().layerAt(st->spp_layers[g]);
            const pxe_dest& pd = st->spp_dests[g][0];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : st->spp_layers[g]);
            const pxe_shim::Slot s = pxe_shim::resolve(pd, pool.pxeOutput(), pool.outputs(), route.pxeOutput(), route.outputs(), plane);
            kernels[g] = pool.pxeKernel();
            ys[g] = s.ptr;
            strides[g] = s.batch_stride;
        }
        PXE_CHECK(pxe_spp(nullptr, input.data(), 0, this->batch(), this->channels(), this->height(), this->width(),
                          st->n_spp, kernels, ys, strides));
        /* a pool with further destinations (two routes read it): copies of its first one */
        for (int g = 0; g < st->n_spp; ++g) {
            for (int k = 1; k < st->n_spp_dests[g]; ++k) {
                auto& pool = this->model().layerAt(st->spp_layers[g]);
                const pxe_dest& pd = st->spp_dests[g][k];
                auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : st->spp_layers[g]);
                const pxe_shim::Slot s = pxe_shim::resolve(pd, pool.pxeOutput(), pool.outputs(), route.pxeOutput(), route.outputs(), plane);
                const float* src = ys[g];
                const int ch = pool.outChannels();
                PXE_CHECK(pxe_concat(nullptr, 1, &src, &strides[g], &ch, s.ptr, s.batch_stride, this->batch(),
                                     this->outHeight(), this->outWidth()));
            }
        }
    }
}
