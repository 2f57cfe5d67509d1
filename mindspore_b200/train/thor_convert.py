"""Conversion of a network / a ``Model`` for the THOR second-order optimizer: ``Dense``, ``Conv2d``, ``Embedding`` and
``EmbeddingLookup`` layers with trainable weights are replaced by their ``*Thor`` forms, which carry the Kronecker
factor state; the new layers share the old layers' parameters (same objects), so an optimizer built on them keeps
working.  ``ConvertModelUtils.convert_to_thor_model`` rebuilds the ``Model`` as a ``ModelThor`` when its optimizer is
THOR.  Parity: mindspore/python/mindspore/train/train_thor/{convert_utils,model_thor}.py.
"""
from ..nn import layer as _layer
from ..nn import layer_ext as _ext
from ..nn.cell import Cell
from .model import Model

__all__ = ["ConvertNetUtils", "ConvertModelUtils", "ModelThor"]


class ConvertNetUtils:
    def __init__(self):
        self._convert_method_map = {_layer.Dense: self._convert_dense, _layer.Embedding: self._convert_embedding,
                                    _layer.EmbeddingLookup: self._convert_embeddinglookup,
                                    _layer.Conv2d: self._convert_conv2d}

    @staticmethod
    def _convert_dense(cell):
        new = _ext.DenseThor(cell.in_channels, cell.out_channels, has_bias=cell.has_bias, activation=cell.activation)
        new.weight = cell.weight
        if cell.has_bias:
            new.bias = cell.bias
        return new

    @staticmethod
    def _convert_embedding(cell):
        new = _ext.EmbeddingThor(cell.vocab_size, cell.embedding_size, padding_idx=cell.padding_idx)
        new.embedding_table = cell.embedding_table
        return new

    @staticmethod
    def _convert_embeddinglookup(cell):
        new = _ext.EmbeddingLookupThor(cell.vocab_size, cell.embedding_size)
        new.embedding_table = cell.embedding_table
        return new

    @staticmethod
    def _convert_conv2d(cell):
        new = _ext.Conv2dThor(cell.in_channels, cell.out_channels, cell.kernel_size, cell.stride, cell.pad_mode,
                              cell.padding, cell.dilation, cell.group, cell.has_bias)
        new.weight = cell.weight
        if cell.has_bias:
            new.bias = cell.bias
        return new

    @staticmethod
    def _need_change(cell, prefix):
        if getattr(cell, "thor", False):
            return False
        if type(cell) in (_layer.Dense, _layer.Conv2d) and cell.weight.requires_grad:
            low = prefix.lower()
            return "rpn_with_loss.rpn_convs_list." not in low and "wide" not in low
        if type(cell) in (_layer.Embedding, _layer.EmbeddingLookup) and cell.embedding_table.requires_grad:
            return True
        return False

    def _convert(self, net, prefix=""):
        for name, sub in list(net.name_cells().items()):
            path = prefix + name
            if self._need_change(sub, path):
                new = self._convert_method_map[type(sub)](sub)
                for p in new.get_parameters(expand=False):           # the factor matrices: named under the layer
                    if not p.name.startswith(path + "."):
                        p.name = path + "." + p.name
                net.insert_child_to_cell(name, new)
                if name in net.__dict__:
                    net.__dict__[name] = new
                if isinstance(getattr(net, "cell_list", None), list):   # SequentialCell runs this list
                    net.cell_list = list(net.name_cells().values())
            else:
                self._convert(sub, path + ".")

    def convert_to_thor_net(self, net):
        """Replaces the layers in place and returns nothing, like the reference."""
        if not isinstance(net, Cell):
            raise TypeError("For 'convert_to_thor_net', 'net' must be a Cell")
        self._convert(net)


class ModelThor(Model):
    """``Model`` whose optimizer is THOR: the factor matrices are refreshed every ``frequency`` steps inside the
    optimizer, so training goes through the ordinary loop."""


class ConvertModelUtils:
    @staticmethod
    def convert_to_thor_model(model, network, loss_fn=None, optimizer=None, metrics=None, amp_level="O0",
                              loss_scale_manager=None, keep_batchnorm_fp32=False):
        name = type(optimizer).__name__
        if name not in ("THOR", "ThorGpu", "ThorAscend"):
            return model
        from ..nn.wrap import TrainOneStepCell
        if isinstance(network, TrainOneStepCell):
            return ModelThor(network=network)
        kwargs = {"network": network, "loss_fn": loss_fn, "optimizer": optimizer, "metrics": metrics,
                  "amp_level": amp_level}
        if loss_scale_manager is not None:
            kwargs["loss_scale_manager"] = loss_scale_manager
        if keep_batchnorm_fp32:
            kwargs["keep_batchnorm_fp32"] = keep_batchnorm_fp32
        return ModelThor(**kwargs)
