/*
 * Body fragment for UpsampleLayer<Device::CUDA>::forward(const V& input), replacing the upsampleGpu call of
 * include/cuda/UpsampleLayer.h:37-38: one pxe_upsample per planned destination -- usually a single one, the channel
 * slot of the route that concatenates the upsampled tensor with a skip connection, so that the route itself runs
 * nothing.
 *
 * Uses the reference's members output_, batch(), channels(), height(), width(), outputs(), outHeight(), outWidth(),
 * stride_, scale_, index(), model(); added by the integration: model().pxePlan(), model().layerAt(i) with pxeOutput()
 * and outputs().
 */
{
    const pxe_step* st = this->model().pxePlan().step(this->index());
    const long long plane = (long long)this->outHeight() * this->outWidth();
    const int n = st != nullptr ? st->n_dests : 1;
    for (int k = 0; k < n; ++k) {
        pxe_shim::Slot s{this->output_.data(), this->outputs()};
        if (st != nullptr) {
            const pxe_dest& pd = st->dests[k];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : this->index());
            s = pxe_shim::resolve(pd, this->output_.data(), this->outputs(), route.pxeOutput(), route.outputs(), plane);
        }
        PXE_CHECK(pxe_upsample(nullptr, input.data(), 0, s.ptr, s.batch_stride, this->batch(), this->channels(),
                               this->height(), this->width(), stride_, scale_));
    }
}
