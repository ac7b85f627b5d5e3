/*
 * Body fragment for ShortcutLayer<Device::CUDA>::forward(const V& input), replacing include/cuda/ShortcutLayer.h:27-33
 * (copy of the input, shortcutGpu with its device synchronisation, activation in place).  A shortcut that the plan
 * folded into the epilogue of the convolution before it runs nothing here.  Otherwise equal shapes take one pass,
 * y = act(alpha * input + beta * from), into up to two planned destinations; unequal shapes keep the reference's
 * three steps on this library's kernels.
 *
 * Uses the reference's members output_, from_, alpha_, beta_, batch(), channels(), height(), width(), outputs(),
 * outChannels(), outHeight(), outWidth(), index(), model(); added by the integration: pxeActivation_ (int),
 * model().pxePlan(), model().layerAt(i) with pxeOutput() and outputs().
 */
{
    const pxe_step* st = this->model().pxePlan().step(this->index());
    if (st == nullptr || (st->op == PXE_STEP_SHORTCUT && st->layer == this->index())) {
        const bool same = from_->outChannels() == this->outChannels() && from_->outHeight() == this->outHeight() &&
                          from_->outWidth() == this->outWidth() && this->channels() == this->outChannels() &&
                          this->height() == this->outHeight() && this->width() == this->outWidth();
        const long long plane = (long long)this->outHeight() * this->outWidth();
        pxe_shim::Slot s[PXE_PLAN_MAX_DESTS] = {{this->output_.data(), this->outputs()}};
        const int n = st != nullptr ? st->n_dests : 1;
        for (int k = 0; k < n && st != nullptr; ++k) {
            const pxe_dest& pd = st->dests[k];
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : this->index());
            s[k] = pxe_shim::resolve(pd, this->output_.data(), this->outputs(), route.pxeOutput(), route.outputs(), plane);
        }
        int stored = 1;                                    /* destinations the kernels below have written */
        if (same) {
            stored = n < 2 ? n : 2;
            PXE_CHECK(pxe_shortcut(nullptr, input.data(), 0, from_->output().data(), 0, s[0].ptr, s[0].batch_stride,
                                   n > 1 ? s[1].ptr : nullptr, n > 1 ? s[1].batch_stride : 0, this->batch(), this->outChannels(),
                                   this->outHeight(), this->outWidth(), alpha_, beta_, pxeActivation_));
        } else {
            /* the general form works in place on a dense tensor: the layer's own, copied to the planned places after */
            this->output_.copy(input);
            PXE_CHECK(pxe_shortcut_general(nullptr, this->batch(), this->width(), this->height(), this->channels(),
                                           from_->output().data(), this->outWidth(), this->outHeight(), this->outChannels(),
                                           alpha_, beta_, this->output_.data()));
            PXE_CHECK(pxe_activate(nullptr, pxeActivation_, this->output_.data(), (size_t)this->batch() * this->outputs()));
            s[0] = pxe_shim::Slot{this->output_.data(), this->outputs()};
            stored = 0;
        }
        const pxe_shim::Slot first = s[0];
        for (int k = stored; k < n && st != nullptr; ++k) {
            const pxe_dest& pd = st->dests[k];
            if (!same && pd.kind == 0) continue;           /* the dense tensor of its own is where the result already is */
            auto& route = this->model().layerAt(pd.kind == 1 ? pd.route : this->index());
            PXE_CHECK(pxe_shim::copy_to(first.ptr, first.batch_stride, this->outChannels(),
                                        pxe_shim::resolve(pd, this->output_.data(), this->outputs(), route.pxeOutput(), route.outputs(), plane),
                                        this->batch(), this->outHeight(), this->outWidth()));
        }
    }
}
