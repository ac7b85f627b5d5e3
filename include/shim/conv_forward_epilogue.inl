/*
 * Body fragment for ConvLayer<Device::CUDA>::forward, replacing include/cuda/ConvLayer.h:284-307 (cuDNN batch-norm
 * inference or addBiasGpu, the preActivation_ copy, activation_->apply) when inferring(); training() keeps the
 * reference's lines.  #include it right after the PX_CHECK_CUDNN that follows cudnnConvolutionForward.
 *
 * Uses the reference's members output_, batch(), outputs(), outHeight(), outWidth(), filters_, batchNorm_, scales_,
 * biases_, rollingMean_, rollingVar_, index(), model(); and, added by the integration: pxeActivation_ (int),
 * model().pxePlan() (const pxe_shim::PlanView&), model().layerAt(i) with pxeOutput() / outputs() / alpha() / beta()
 * / pxeActivation() on the layers it returns.
 */
{
    const pxe_step* st = this->model().pxePlan().step(this->index());
    if (st != nullptr && !st->head_raw) {          /* head_raw: the YOLO decode applies bias + logistic itself */
        const long long plane = (long long)this->outHeight() * this->outWidth();
        pxe_epilogue_desc d{};
        d.x = this->output_.data();
        d.x_batch_stride = this->outputs();
        d.batch = this->batch();
        d.channels = filters_;
        d.height = this->outHeight();
        d.width = this->outWidth();
        if (batchNorm_) {
            d.gamma = scales_.data();
            d.beta = biases_.data();
            d.mean = rollingMean_.data();
            d.var = rollingVar_.data();
            d.eps = 0.00001f;
            d.eps_mode = PXE_BN_EPS_CUDNN;
        } else {
            d.bias = biases_.data();
        }
        d.act = pxeActivation_;
        /* the layer whose value this step defines: this conv, or the shortcut folded into it */
        const int out_layer = st->fused_shortcut >= 0 ? st->fused_shortcut : this->index();
        auto& out = this->model().layerAt(out_layer);
        if (st->fused_shortcut >= 0) {
            auto& from = this->model().layerAt(st->inputs[1]);
            d.residual = from.pxeOutput();
            d.residual_batch_stride = from.outputs();
            d.res_alpha = out.alpha();
            d.res_beta = out.beta();
            d.res_act = out.pxeActivation();
        }
        if (st->fused_pool < 0 || st->keep_full) {
            for (int k = 0; k < st->n_dests && k < 2; ++k) {
                const pxe_dest& pd = st->dests[k];
                auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : out_layer);
                const pxe_shim::Slot s = pxe_shim::resolve(pd, out.pxeOutput(), out.outputs(), route.pxeOutput(),
                                                           route.outputs(), plane);
                if (k == 0) { d.y = s.ptr; d.y_batch_stride = s.batch_stride; }
                else { d.y2 = s.ptr; d.y2_batch_stride = s.batch_stride; }
            }
        }
        if (st->fused_pool >= 0) {
            auto& pool = this->model().layerAt(st->fused_pool);
            const pxe_dest& pd = st->pool_dests[0];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : st->fused_pool);
            const pxe_shim::Slot s = pxe_shim::resolve(pd, pool.pxeOutput(), pool.outputs(), route.pxeOutput(),
                                                       route.outputs(), (long long)pool.outHeight() * pool.outWidth());
            d.pool_kernel = 2;
            d.pool_stride = 2;
            d.pool_padding = pool.padding();
            d.y_pool = s.ptr;
            d.y_pool_batch_stride = s.batch_stride;
        }
        PXE_CHECK(pxe_conv_epilogue(nullptr, &d));
        for (int k = 1; st->fused_pool >= 0 && k < st->n_pool_dests; ++k) {   /* the pooled tensor, stored more than once */
            auto& pool = this->model().layerAt(st->fused_pool);
            const pxe_dest& pd = st->pool_dests[k];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : st->fused_pool);
            PXE_CHECK(pxe_shim::copy_to(d.y_pool, d.y_pool_batch_stride, filters_,
                                        pxe_shim::resolve(pd, pool.pxeOutput(), pool.outputs(), route.pxeOutput(), route.outputs(),
                                                          (long long)pool.outHeight() * pool.outWidth()),
                                        this->batch(), pool.outHeight(), pool.outWidth()));
        }
        for (int k = 2; k < st->n_dests && d.y != nullptr; ++k) {          /* read by more than two routes: copies */
            const pxe_dest& pd = st->dests[k];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : out_layer);
            PXE_CHECK(pxe_shim::copy_to(d.y, d.y_batch_stride, filters_,
                                        pxe_shim::resolve(pd, out.pxeOutput(), out.outputs(), route.pxeOutput(), route.outputs(), plane),
                                        this->batch(), this->outHeight(), this->outWidth()));
        }
    }
}
