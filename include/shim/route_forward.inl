/*
 * Body fragment for RouteLayer<Device::CUDA>::forward, replacing the copy loop of include/cuda/RouteLayer.h:25-43.
 * When the plan redirected every producer into this route's buffer (PXE_STEP_ALIAS) nothing runs; otherwise one
 * pxe_concat gathers the sources (instead of batch() x fan-in blocking cudaMemcpy calls).
 *
 * Uses the reference's members output_, batch(), outHeight(), outWidth(), layers_ (the source layers), index(),
 * model(); added by the integration: model().pxePlan().
 */
{
    const pxe_step* st = this->model().pxePlan().step(this->index());
    if (st == nullptr || st->op != PXE_STEP_ALIAS) {
        const int n = (int)layers_.size();
        std::vector<const float*> srcs((size_t)n);
        std::vector<long long> strides((size_t)n);
        std::vector<int> channels((size_t)n);
        for (int i = 0; i < n; ++i) {
            srcs[i] = layers_[i]->output().data();
            strides[i] = layers_[i]->outputs();
            channels[i] = layers_[i]->outChannels();
        }
        PXE_CHECK(pxe_concat(nullptr, n, srcs.data(), strides.data(), channels.data(), this->output_.data(),
                             this->outputs(), this->batch(), this->outHeight(), this->outWidth()));
    }
}
