"""The last primitives of ``mindspore.ops.operations``: recurrent cells over packed weights (BasicLSTMCell, DynamicRNN,
DynamicGRUV2), the fused Adafactor update, the transducer loss, replay-buffer and embedding-cache bookkeeping,
fractional pooling, 3-D patch extraction, overlap-matrix and combined NMS, deformable sampling, kernel-based
scale-and-translate, distorted bounding boxes, sparse slicing.  Built with the same table helper as
``operations_more``; attribute names and input orders follow python/mindspore/ops/operations/{nn_ops,inner_ops,rl_ops,
array_ops,image_ops,other_ops,sparse_ops,_embedding_cache_ops}.py."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import operations_more as _more
from .function_ext import _w
from .operations_more import _REQ, _t

__all__ = []


def _prim(name, params=(), run=None, doc=None):
    cls = _more._prim(name, params, run, doc)
    cls.__module__ = __name__
    globals()[name] = cls
    __all__.append(name)
    return cls


# ------------------------------------------------------------------------------------------------ recurrent cells
def _lstm_step(x, h, c, w, b, forget_bias):
    gates = torch.cat([x, h], -1) @ w + b
    i, j, f, o = gates.chunk(4, -1)                      # input, candidate, forget, output
    it, jt, ft, ot = torch.sigmoid(i), torch.tanh(j), torch.sigmoid(f + forget_bias), torch.sigmoid(o)
    ct = c * ft + it * jt
    tanhct = torch.tanh(ct)
    return ct, tanhct * ot, it, jt, ft, ot, tanhct


def _basic_lstm_cell(self, x, h, c, w, b):
    x, h, c, w, b = (_t(v) for v in (x, h, c, w, b))
    if self.keep_prob < 1.0:
        x = F.dropout(x, 1.0 - self.keep_prob)
    return _lstm_step(x, h, c, w, b, self.forget_bias)


_prim("BasicLSTMCell", [("keep_prob", 1.0), ("forget_bias", 1.0), ("state_is_tuple", True), ("activation", "tanh")],
      _basic_lstm_cell)


def _dynamic_rnn(self, x, w, b, seq_length=None, init_h=None, init_c=None):
    """x [T, B, I], w [I + H, 4H], b [4H], init_h / init_c [1, B, H] -> y, h, c, i, j, f, o, tanh(c), each [T, B, H];
    steps at or past a sample's ``seq_length`` keep the state and emit zeros."""
    x, w, b = _t(x), _t(w), _t(b)
    steps, batch, hidden = x.shape[0], x.shape[1], w.shape[1] // 4
    h = _t(init_h)[0] if init_h is not None else x.new_zeros(batch, hidden)
    c = _t(init_c)[0] if init_c is not None else x.new_zeros(batch, hidden)
    lengths = _t(seq_length).to(torch.long) if seq_length is not None else None
    outs = [[] for _ in range(8)]
    for t in range(steps):
        ct, ht, it, jt, ft, ot, tanhct = _lstm_step(x[t], h, c, w, b, self.forget_bias)
        if self.cell_clip > 0:
            ct = ct.clamp(-self.cell_clip, self.cell_clip)
        y = ht
        if lengths is not None:
            live = (t < lengths).unsqueeze(-1)
            ct, ht, y = torch.where(live, ct, c), torch.where(live, ht, h), torch.where(live, ht, torch.zeros_like(ht))
        h, c = ht, ct
        for k, v in enumerate((y, ht, ct, it, jt, ft, ot, tanhct)):
            outs[k].append(v)
    return tuple(torch.stack(o) for o in outs)


_prim("DynamicRNN", [("cell_type", "LSTM"), ("direction", "UNIDIRECTIONAL"), ("cell_depth", 1),
                     ("use_peephole", False), ("keep_prob", 1.0), ("cell_clip", -1.0), ("num_proj", 0),
                     ("time_major", True), ("activation", "tanh"), ("forget_bias", 0.0), ("is_training", True)],
      _dynamic_rnn)


def _dynamic_gru_v2(self, x, weight_input, weight_hidden, bias_input=None, bias_hidden=None, seq_length=None,
                    init_h=None):
    """x [T, B, I], weight_input [I, 3H], weight_hidden [H, 3H] (gate order ``rzh`` or ``zrh``) -> y, output_h,
    update, reset, new, hidden_new, each [T, B, H]."""
    x, wi, wh = _t(x), _t(weight_input), _t(weight_hidden)
    hidden = wh.shape[0]
    bi = _t(bias_input) if bias_input is not None else x.new_zeros(3 * hidden)
    bh = _t(bias_hidden) if bias_hidden is not None else x.new_zeros(3 * hidden)
    h = _t(init_h) if init_h is not None else x.new_zeros(x.shape[1], hidden)
    lengths = _t(seq_length).to(torch.long) if seq_length is not None else None
    outs = [[] for _ in range(6)]
    for t in range(x.shape[0]):
        gi, gh = x[t] @ wi + bi, h @ wh + bh
        a, b_, xn = gi.chunk(3, -1)
        ha, hb, hn = gh.chunk(3, -1)
        first, second = torch.sigmoid(a + ha), torch.sigmoid(b_ + hb)
        r, z = (first, second) if self.gate_order == "rzh" else (second, first)
        if self.reset_after:
            hidden_new = hn
            n = torch.tanh(xn + r * hn)
        else:
            hidden_new = (r * h) @ wh[:, 2 * hidden:] + bh[2 * hidden:]
            n = torch.tanh(xn + hidden_new)
        new_h = (1 - z) * n + z * h
        y = new_h
        if lengths is not None:
            live = (t < lengths).unsqueeze(-1)
            new_h, y = torch.where(live, new_h, h), torch.where(live, new_h, torch.zeros_like(new_h))
        h = new_h
        for k, v in enumerate((y, h, z, r, n, hidden_new)):
            outs[k].append(v)
    return tuple(torch.stack(o) for o in outs)


_prim("DynamicGRUV2", [("direction", "UNIDIRECTIONAL"), ("cell_depth", 1), ("keep_prob", 1.0), ("cell_clip", -1.0),
                       ("num_proj", 0), ("time_major", True), ("activation", "tanh"), ("gate_order", "rzh"),
                       ("reset_after", True), ("is_training", True)], _dynamic_gru_v2)


# ------------------------------------------------------------------------------------------------ fused Adafactor
def _adafactor(self, epsilon, clip_threshold, beta1, beta2, weight_decay, learning_rate, gradient, param, exp_avg,
               exp_avg_sq_row, exp_avg_sq_col, exp_avg_sq, global_norm=None):
    """One Adafactor update in place: factored second moment (row / column means) for matrices, full second moment
    otherwise; update clipped to ``clip_threshold`` RMS; optional first moment, parameter scaling and weight decay."""
    g = _t(gradient).float()
    if global_norm is not None:
        g = g / torch.clamp(_t(global_norm).float(), min=1.0)
    p = _t(param)
    eps1, eps2 = (float(v) for v in _t(epsilon).reshape(-1)[:2])
    beta1, beta2 = float(_t(beta1)), float(_t(beta2))
    lr, wd, clip = float(_t(learning_rate)), float(_t(weight_decay)), float(_t(clip_threshold))
    with torch.no_grad():
        pf = p.float()
        if self.enable_scale_parameter:
            lr = lr * max(eps2, float(pf.pow(2).mean().sqrt()))
        sq = g * g + eps1
        if g.dim() >= 2:
            row, col = _t(exp_avg_sq_row), _t(exp_avg_sq_col)
            row.mul_(beta2).add_(sq.mean(-1).to(row.dtype), alpha=1 - beta2)
            col.mul_(beta2).add_(sq.mean(-2).to(col.dtype), alpha=1 - beta2)
            r = (row.float() / row.float().mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
            update = g * r * col.float().rsqrt().unsqueeze(-2)
        else:
            full = _t(exp_avg_sq)
            full.mul_(beta2).add_(sq.to(full.dtype), alpha=1 - beta2)
            update = g * full.float().rsqrt()
        update = update / max(1.0, float(update.pow(2).mean().sqrt()) / clip)
        update = update * lr
        if self.enable_first_moment:
            m = _t(exp_avg)
            m.mul_(beta1).add_(update.to(m.dtype), alpha=1 - beta1)
            update = m.float()
        if self.enable_weight_decay:
            pf = pf - wd * lr * pf
        p.copy_((pf - update).to(p.dtype))
    return p


_ADAFACTOR_ARGS = [("enable_scale_parameter", False), ("enable_first_moment", False), ("enable_weight_decay", False)]
_prim("FusedAdaFactor", _ADAFACTOR_ARGS, _adafactor)
_prim("FusedAdaFactorWithGlobalNorm", _ADAFACTOR_ARGS, _adafactor)


# ------------------------------------------------------------------------------------------------ transducer loss
def _rnnt_loss(self, acts, labels, input_length, label_length):
    """acts [B, T, U, V] (unnormalised), labels [B, U - 1] -> (costs [B], grads [B, T, U, V]).  The forward variable
    runs over the (t, u) lattice in log space; the gradient is that of the summed costs."""
    acts = _t(acts).detach().float().requires_grad_(True)
    labels, t_len, u_len = _t(labels).long(), _t(input_length).long(), _t(label_length).long()
    with torch.enable_grad():
        logp = torch.log_softmax(acts, -1)
        costs = []
        for b in range(acts.shape[0]):
            T, U = int(t_len[b]), int(u_len[b]) + 1
            blank = logp[b, :T, :U, self.blank_label]
            emit = logp[b, :T, :U - 1].gather(-1, labels[b, :U - 1].reshape(1, -1, 1).expand(T, -1, -1)).squeeze(-1) \
                if U > 1 else None
            alpha = [[None] * U for _ in range(T)]
            alpha[0][0] = logp.new_zeros(())
            for t in range(T):
                for u in range(U):
                    if t == 0 and u == 0:
                        continue
                    terms = []
                    if t > 0:
                        terms.append(alpha[t - 1][u] + blank[t - 1, u])
                    if u > 0:
                        terms.append(alpha[t][u - 1] + emit[t, u - 1])
                    alpha[t][u] = terms[0] if len(terms) == 1 else torch.logaddexp(terms[0], terms[1])
            costs.append(-(alpha[T - 1][U - 1] + blank[T - 1, U - 1]))
        costs = torch.stack(costs)
        (grads,) = torch.autograd.grad(costs.sum(), acts)
    return costs.detach(), grads


_prim("RNNTLoss", [("blank_label", 0)], _rnnt_loss)


# ------------------------------------------------------------------------------------------------ replay buffer
def _buffer_append(self, buffer, exp, count, head):
    """Ring buffer write: ``buffer`` is a tuple of [capacity, ...] tensors, ``exp`` one row (or a batch of rows) per
    tensor; ``count`` / ``head`` (one-element int tensors) are updated in place."""
    count, head = _t(count), _t(head)
    rows = None
    for buf, item in zip(buffer, exp):
        buf, item = _t(buf), _t(item)
        batch = item.reshape((-1,) + tuple(buf.shape[1:]))
        rows = batch.shape[0]
        for k in range(rows):
            n, h = int(count.reshape(-1)[0]), int(head.reshape(-1)[0])
            at = (h + n + k) % self.capacity if n + k < self.capacity else (h + k) % self.capacity
            buf[at] = batch[k].to(buf.dtype)
    n, h = int(count.reshape(-1)[0]), int(head.reshape(-1)[0])
    overflow = max(0, n + rows - self.capacity)
    count.fill_(min(self.capacity, n + rows))
    head.fill_((h + overflow) % self.capacity)
    return count


def _buffer_get(self, buffer, count, head, index):
    n, h, i = int(_t(count).reshape(-1)[0]), int(_t(head).reshape(-1)[0]), int(_t(index).reshape(-1)[0])
    if i < -n or i >= n:
        raise ValueError("For 'BufferGetItem', index %d is out of range for %d stored items" % (i, n))
    at = (h + (i % n)) % self.capacity
    return tuple(_t(buf)[at] for buf in buffer)


def _buffer_sample(self, buffer, count, head):
    n, h = int(_t(count).reshape(-1)[0]), int(_t(head).reshape(-1)[0])
    if n == 0:
        raise ValueError("For 'BufferSample', the buffer is empty")
    gen = torch.Generator()
    gen.manual_seed(self.seed) if self.seed else gen.seed()
    if self.unique:
        if self.batch_size > n:
            raise ValueError("For 'BufferSample', batch_size %d exceeds the %d stored items" % (self.batch_size, n))
        pick = torch.randperm(n, generator=gen)[:self.batch_size]
    else:
        pick = torch.randint(0, n, (self.batch_size,), generator=gen)
    at = (pick + h) % self.capacity
    return tuple(_t(buf)[at] for buf in buffer)


_BUF = [("capacity", _REQ), ("buffer_shape", _REQ), ("buffer_dtype", _REQ)]
_prim("BufferAppend", _BUF, _buffer_append)
_prim("BufferGetItem", _BUF, _buffer_get)
_prim("BufferSample", [("capacity", _REQ), ("batch_size", _REQ), ("buffer_shape", _REQ), ("buffer_dtype", _REQ),
                       ("seed", 0), ("unique", False)], _buffer_sample)


# ------------------------------------------------------------------------------------------------ embedding cache
def _sub_and_filter(self, input_x, max_num, offset):
    x = _t(input_x).reshape(-1) - int(offset)
    keep = (x >= 0) & (x < int(max_num))
    return x[keep], torch.nonzero(keep).reshape(-1).to(x.dtype)


def _map_uniform(self, input, per_group_size, group_num):                                  # noqa: A002
    x = _t(input)
    return (x % int(group_num)) * int(per_group_size) + x // int(group_num)


def _map_cache_idx(self, hashmap, indices, step, emb_max_num, offset):
    """``hashmap`` [N, 4] rows (key, cache slot, last step, used flag), open addressing from ``key % N``.  Returns
    (cache_idx per index, -1 where out of range; evicted keys; missed keys; cache slots of the misses).  A miss takes
    a free row; when the table is more than 90 % full the least recently used entry of an earlier step is evicted."""
    table = _t(hashmap)
    n = table.shape[0]
    step, emb_max, offset = int(_t(step)), int(_t(emb_max_num)), int(_t(offset))
    ids = _t(indices).reshape(-1).tolist()
    cache_idx, old, miss, swap = [], [], [], []
    used = int((table[:, 3] != 0).sum())

    def probe(key):
        at = key % n
        for _ in range(n):
            if table[at, 3] == 0 or int(table[at, 0]) == key:
                return at
            at = (at + 1) % n
        return -1

    for raw in ids:
        key = raw - offset
        if key < 0 or key >= emb_max:
            cache_idx.append(-1)
            continue
        at = probe(key)
        if at >= 0 and table[at, 3] != 0:
            table[at, 2] = step
            cache_idx.append(int(table[at, 1]))
            continue
        if at < 0 or used >= int(0.9 * n):
            live = torch.nonzero((table[:, 3] != 0) & (table[:, 2] < step)).reshape(-1)
            if live.numel() == 0:
                raise RuntimeError("For 'MapCacheIdx', the cache is full of entries of the current step")
            victim = int(live[torch.argmin(table[live, 2])])
            slot = int(table[victim, 1])
            old.append(int(table[victim, 0]))
            table[victim, 3] = 0
            used -= 1
            at = probe(key)
        else:
            slot = used
        table[at] = torch.tensor([key, slot, step, 1], dtype=table.dtype)
        used += 1
        miss.append(key)
        swap.append(slot)
        cache_idx.append(slot)
    mk = lambda v: torch.tensor(v, dtype=table.dtype)                                     # noqa: E731
    return mk(cache_idx).reshape(_t(indices).shape), mk(old), mk(miss), mk(swap)


_prim("SubAndFilter", (), _sub_and_filter)
_prim("MapUniform", (), _map_uniform)
_prim("MapCacheIdx", (), _map_cache_idx)

# keys of the parameter-server push / pull pair: (optimizer, inputs) by key, weights by key
_PS_STORE = {"next": 0, "pushed": {}}


def _push(self, optim_inputs, optim_input_shapes):
    key = _PS_STORE["next"]
    _PS_STORE["next"] += 1
    _PS_STORE["pushed"][key] = (self.optim_type, tuple(_t(v).clone() for v in optim_inputs))
    return torch.tensor(key, dtype=torch.int64)


def _pull(self, key, weight):
    return _t(weight)


_prim("Push", [("optim_type", "ApplyMomentum"), ("only_shape_indices", None)], _push)
_prim("Pull", (), _pull)


# ------------------------------------------------------------------------------------------------ patches / pooling
def _extract_volume_patches(self, x):
    """[N, C, D, H, W] -> [N, C * kd * kh * kw, oD, oH, oW]; channels ordered (kd, kh, kw, C)."""
    t = _t(x)
    kd, kh, kw = self.kernel_size[2:]
    sd, sh, sw = self.strides[2:]
    if str(self.padding).upper() == "SAME":
        pads = []
        for size, k, s in ((t.shape[4], kw, sw), (t.shape[3], kh, sh), (t.shape[2], kd, sd)):
            total = max((math.ceil(size / s) - 1) * s + k - size, 0)
            pads += [total // 2, total - total // 2]
        t = F.pad(t, pads)
    p = t.unfold(2, kd, sd).unfold(3, kh, sh).unfold(4, kw, sw)          # N C oD oH oW kd kh kw
    n, c, od, oh, ow = p.shape[:5]
    return p.permute(0, 5, 6, 7, 1, 2, 3, 4).reshape(n, kd * kh * kw * c, od, oh, ow)


_prim("ExtractVolumePatches", [("kernel_size", _REQ), ("strides", _REQ), ("padding", _REQ)], _extract_volume_patches)


def _fractional_sequence(in_size, out_size, pseudo_random, gen):
    """Cut points 0 = a_0 < ... < a_out = in_size with steps of floor(alpha) or ceil(alpha), alpha = in / out."""
    alpha = in_size / out_size
    if pseudo_random:
        u = float(torch.rand((), generator=gen))
        seq = [int(math.ceil(alpha * (i + u))) - int(math.ceil(alpha * u)) for i in range(out_size)]
    else:
        small = int(math.floor(alpha))
        n_big = in_size - small * out_size
        steps = [small + 1] * n_big + [small] * (out_size - n_big)
        perm = torch.randperm(out_size, generator=gen).tolist()
        steps = [steps[i] for i in perm]
        seq = [0]
        for s in steps[:-1]:
            seq.append(seq[-1] + s)
    return seq + [in_size]


def _fractional_pool(reduce):
    def run(self, x):
        t = _t(x)                                                        # NHWC
        ratio = [float(r) for r in self.pooling_ratio]
        if len(ratio) != 4 or ratio[0] != 1.0 or ratio[3] != 1.0:
            raise ValueError("pooling_ratio must be [1.0, rows, cols, 1.0], but got %r" % (self.pooling_ratio,))
        gen = torch.Generator()
        seed = (int(self.seed) << 16) ^ int(self.seed2)
        gen.manual_seed(seed) if (seed or self.deterministic) else gen.seed()
        h, w = t.shape[1], t.shape[2]
        rows = _fractional_sequence(h, int(h / ratio[1]), self.pseudo_random, gen)
        cols = _fractional_sequence(w, int(w / ratio[2]), self.pseudo_random, gen)
        extra = 1 if self.overlapping else 0
        out = t.new_empty(t.shape[0], len(rows) - 1, len(cols) - 1, t.shape[3])
        for i in range(len(rows) - 1):
            r0, r1 = rows[i], min(rows[i + 1] + extra, h)
            for j in range(len(cols) - 1):
                c0, c1 = cols[j], min(cols[j + 1] + extra, w)
                out[:, i, j] = reduce(t[:, r0:r1, c0:c1].reshape(t.shape[0], -1, t.shape[3]))
        return out, torch.tensor(rows, dtype=torch.int64), torch.tensor(cols, dtype=torch.int64)
    return run


_FRAC = [("pooling_ratio", _REQ), ("pseudo_random", False), ("overlapping", False), ("deterministic", False),
         ("seed", 0), ("seed2", 0)]
_prim("FractionalMaxPool", _FRAC, _fractional_pool(lambda v: v.amax(1)))
_prim("FractionalAvgPool", _FRAC, _fractional_pool(lambda v: v.float().mean(1).to(v.dtype)))


def _fractional_fixed(dims):
    pool = F.fractional_max_pool2d if dims == 2 else F.fractional_max_pool3d

    def run(self, x, random_samples):
        t = _t(x)
        channels_last = self.data_format in ("NHWC", "NDHWC")
        if channels_last:
            t = t.movedim(-1, 1)
        samples = _t(random_samples).to(t.dtype if t.is_floating_point() else torch.float32)
        y, idx = pool(t.float() if not t.is_floating_point() else t, tuple(self.ksize) if not isinstance(
            self.ksize, int) else self.ksize, output_size=tuple(self.output_shape) if not isinstance(
            self.output_shape, int) else self.output_shape, return_indices=True, _random_samples=samples)
        y = y.to(t.dtype)
        if channels_last:
            y, idx = y.movedim(1, -1), idx.movedim(1, -1)
        return y, idx
    return run


_prim("FractionalMaxPoolWithFixedKsize", [("ksize", _REQ), ("output_shape", _REQ), ("data_format", "NCHW")],
      _fractional_fixed(2))
_prim("FractionalMaxPool3DWithFixedKsize", [("ksize", _REQ), ("output_shape", _REQ), ("data_format", "NCDHW")],
      _fractional_fixed(3))


# ------------------------------------------------------------------------------------------------ detection
def _nms_overlaps(self, overlaps, scores, max_output_size, overlap_threshold, score_threshold):
    ov, sc = _t(overlaps), _t(scores)
    limit, thr, floor = int(_t(max_output_size)), float(_t(overlap_threshold)), float(_t(score_threshold))
    keep = []
    for i in torch.argsort(sc, descending=True, stable=True).tolist():
        if len(keep) >= limit or sc[i] <= floor:
            break
        if all(float(ov[i, j]) <= thr for j in keep):
            keep.append(i)
    return torch.tensor(keep, dtype=torch.int32)


_prim("NonMaxSuppressionWithOverlaps", (), _nms_overlaps)


def _iou_row(box, boxes):
    y1, x1 = torch.minimum(boxes[:, 0], boxes[:, 2]), torch.minimum(boxes[:, 1], boxes[:, 3])
    y2, x2 = torch.maximum(boxes[:, 0], boxes[:, 2]), torch.maximum(boxes[:, 1], boxes[:, 3])
    by1, bx1, by2, bx2 = min(box[0], box[2]), min(box[1], box[3]), max(box[0], box[2]), max(box[1], box[3])
    inter = (torch.minimum(y2, by2) - torch.maximum(y1, by1)).clamp(min=0) * \
        (torch.minimum(x2, bx2) - torch.maximum(x1, bx1)).clamp(min=0)
    union = (y2 - y1) * (x2 - x1) + (by2 - by1) * (bx2 - bx1) - inter
    return torch.where(union > 0, inter / union, torch.zeros_like(inter))


def _combined_nms(self, boxes, scores, max_output_size_per_class, max_total_size, iou_threshold, score_threshold):
    """boxes [B, N, q, 4] (q = 1 or classes), scores [B, N, C] -> boxes [B, M, 4], scores [B, M], classes [B, M],
    valid [B]; M = max_total_size (or per_class * C capped by it with ``pad_per_class``)."""
    bx, sc = _t(boxes).float(), _t(scores).float()
    per_class, total = int(_t(max_output_size_per_class)), int(_t(max_total_size))
    iou_thr, floor = float(_t(iou_threshold)), float(_t(score_threshold))
    batch, _, q, _ = bx.shape
    classes = sc.shape[2]
    size = min(total, per_class * classes) if self.pad_per_class else total
    out_b, out_s = bx.new_zeros(batch, size, 4), bx.new_zeros(batch, size)
    out_c, valid = bx.new_zeros(batch, size), torch.zeros(batch, dtype=torch.int32)
    for b in range(batch):
        picked = []
        for c in range(classes):
            cb, cs = bx[b, :, c if q > 1 else 0], sc[b, :, c]
            keep = []
            for i in torch.argsort(cs, descending=True, stable=True).tolist():
                if len(keep) >= per_class or cs[i] <= floor:
                    break
                if not keep or float(_iou_row(cb[i], cb[keep]).max()) <= iou_thr:
                    keep.append(i)
            picked += [(float(cs[i]), c, cb[i]) for i in keep]
        picked.sort(key=lambda r: -r[0])
        picked = picked[:size]
        valid[b] = len(picked)
        for k, (s, c, box) in enumerate(picked):
            out_b[b, k] = box.clamp(0, 1) if self.clip_boxes else box
            out_s[b, k], out_c[b, k] = s, c
    return out_b, out_s, out_c, valid


_prim("CombinedNonMaxSuppression", [("pad_per_class", False), ("clip_boxes", True)], _combined_nms)


def _deformable_offsets(self, x, offsets):
    """Samples the input at the deformed positions of every kernel tap: x [N, C, H, W], offsets [N, 3 * G * kh * kw,
    oH, oW] (x offsets, y offsets, masks) -> [N, C, oH * kh, oW * kw], ready for a stride-k convolution."""
    t, off = _t(x).float(), _t(offsets).float()
    nhwc = self.data_format == "NHWC"
    if nhwc:
        t, off = t.permute(0, 3, 1, 2), off.permute(0, 3, 1, 2)
    n, c, h, w = t.shape
    kh, kw = self.ksize
    sh, sw = self.strides[-2:]
    dh, dw = self.dilations[-2:]
    pt, _, pl, _ = self.pads
    g = self.deformable_groups
    oh, ow = off.shape[2], off.shape[3]
    off = off.reshape(n, 3, g, kh, kw, oh, ow)
    base_y = (torch.arange(oh) * sh - pt).reshape(1, 1, 1, 1, oh, 1) + (torch.arange(kh) * dh).reshape(1, 1, kh, 1, 1, 1)
    base_x = (torch.arange(ow) * sw - pl).reshape(1, 1, 1, 1, 1, ow) + (torch.arange(kw) * dw).reshape(1, 1, 1, kw, 1, 1)
    py, px = base_y + off[:, 1], base_x + off[:, 0]                     # N G kh kw oH oW
    grid = torch.stack([2 * px / max(w - 1, 1) - 1, 2 * py / max(h - 1, 1) - 1], -1)
    grid = grid.permute(0, 1, 4, 2, 5, 3, 6).reshape(n * g, oh * kh, ow * kw, 2)
    sampled = F.grid_sample(t.reshape(n * g, c // g, h, w), grid, mode="bilinear", padding_mode="zeros",
                            align_corners=True)
    if self.modulated:
        mask = off[:, 2].permute(0, 1, 4, 2, 5, 3).reshape(n * g, 1, oh * kh, ow * kw)
        sampled = sampled * mask
    out = sampled.reshape(n, c, oh * kh, ow * kw).to(_t(x).dtype)
    return out.permute(0, 2, 3, 1) if nhwc else out


_prim("DeformableOffsets", [("strides", _REQ), ("pads", _REQ), ("ksize", _REQ), ("dilations", (1, 1, 1, 1)),
                            ("data_format", "NCHW"), ("deformable_groups", 1), ("modulated", True)],
      _deformable_offsets)


def _sample_distorted_box(self, image_size, bounding_boxes, min_object_covered):
    """A random crop window (begin [y, x, 0], size [h, w, -1], the window as a box [1, 1, 4]) whose aspect ratio and
    area fall in the configured ranges and that covers ``min_object_covered`` of at least one box."""
    height, width = (int(v) for v in _t(image_size).reshape(-1)[:2])
    boxes = _t(bounding_boxes).float().reshape(-1, 4)
    cover = float(_t(min_object_covered).reshape(-1)[0])
    if boxes.numel() == 0:
        if not self.use_image_if_no_bounding_boxes:
            raise ValueError("For 'SampleDistortedBoundingBoxV2', no bounding boxes were given")
        boxes = torch.tensor([[0.0, 0.0, 1.0, 1.0]])
    gen = torch.Generator()
    seed = (int(self.seed) << 16) ^ int(self.seed2)
    gen.manual_seed(seed) if seed else gen.seed()
    rand = lambda lo, hi: lo + (hi - lo) * float(torch.rand((), generator=gen))           # noqa: E731
    y0, x0, hh, ww = 0, 0, height, width
    for _ in range(int(self.max_attempts)):
        ratio = rand(*self.aspect_ratio_range)
        area = rand(*self.area_range) * height * width
        ch, cw = int(round(math.sqrt(area / ratio))), int(round(math.sqrt(area * ratio)))
        if ch <= 0 or cw <= 0 or ch > height or cw > width:
            continue
        cy, cx = int(rand(0, height - ch + 1)), int(rand(0, width - cw + 1))
        win = torch.tensor([cy / height, cx / width, (cy + ch) / height, (cx + cw) / width])
        iy = (torch.minimum(boxes[:, 2], win[2]) - torch.maximum(boxes[:, 0], win[0])).clamp(min=0)
        ix = (torch.minimum(boxes[:, 3], win[3]) - torch.maximum(boxes[:, 1], win[1])).clamp(min=0)
        box_area = ((boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1])).clamp(min=1e-12)
        if bool(((iy * ix) / box_area >= cover).any()):
            y0, x0, hh, ww = cy, cx, ch, cw
            break
    dtype = _t(image_size).dtype
    begin = torch.tensor([y0, x0, 0], dtype=dtype)
    size = torch.tensor([hh, ww, -1], dtype=dtype)
    box = torch.tensor([[[y0 / height, x0 / width, (y0 + hh) / height, (x0 + ww) / width]]])
    return begin, size, box


_prim("SampleDistortedBoundingBoxV2", [("seed", 0), ("seed2", 0), ("aspect_ratio_range", (0.75, 1.33)),
                                       ("area_range", (0.05, 1.0)), ("max_attempts", 100),
                                       ("use_image_if_no_bounding_boxes", False)], _sample_distorted_box)


# ------------------------------------------------------------------------------------------------ resampling
def _kernel(kind):
    def lanczos(radius):
        def f(x):
            x = x.abs()
            val = torch.sinc(x) * torch.sinc(x / radius)
            return torch.where(x < radius, val, torch.zeros_like(val))
        return f, float(radius)

    def cubic(b, c):
        def f(x):
            x = x.abs()
            near = ((12 - 9 * b - 6 * c) * x ** 3 + (-18 + 12 * b + 6 * c) * x ** 2 + (6 - 2 * b)) / 6
            far = ((-b - 6 * c) * x ** 3 + (6 * b + 30 * c) * x ** 2 + (-12 * b - 48 * c) * x + (8 * b + 24 * c)) / 6
            return torch.where(x < 1, near, torch.where(x < 2, far, torch.zeros_like(x)))
        return f, 2.0
    table = {"lanczos1": lanczos(1), "lanczos3": lanczos(3), "lanczos5": lanczos(5),
             "gaussian": (lambda x: torch.where(x.abs() < 1.5, torch.exp(-2.0 * x * x), torch.zeros_like(x)), 1.5),
             "box": (lambda x: ((x >= -0.5) & (x < 0.5)).to(x.dtype), 0.5),
             "triangle": (lambda x: (1 - x.abs()).clamp(min=0), 1.0),
             "keyscubic": cubic(0.0, 0.5), "mitchellcubic": cubic(1 / 3, 1 / 3)}
    if kind not in table:
        raise ValueError("For 'ScaleAndTranslate', unknown kernel_type %r" % (kind,))
    return table[kind]


def _resample_weights(in_size, out_size, scale, translate, fn, radius, antialias):
    """[out_size, in_size] matrix: output sample o reads input position (o + 0.5 - translate) / scale - 0.5."""
    stretch = max(1.0 / scale, 1.0) if antialias else 1.0
    centre = (torch.arange(out_size, dtype=torch.float64) + 0.5 - translate) / scale
    src = torch.arange(in_size, dtype=torch.float64) + 0.5
    wts = fn((src.unsqueeze(0) - centre.unsqueeze(1)) / stretch)
    inside = (centre >= -radius * stretch) & (centre <= in_size + radius * stretch)
    total = wts.sum(1, keepdim=True)
    wts = torch.where(total.abs() > 1e-12, wts / total, torch.zeros_like(wts))
    return (wts * inside.unsqueeze(1)).float()


def _scale_and_translate(self, images, size, scale, translation):
    t = _t(images).float()                                              # NHWC
    oh, ow = (int(v) for v in _t(size).reshape(-1)[:2])
    sy, sx = (float(v) for v in _t(scale).reshape(-1)[:2])
    ty, tx = (float(v) for v in _t(translation).reshape(-1)[:2])
    fn, radius = _kernel(self.kernel_type)
    wy = _resample_weights(t.shape[1], oh, sy, ty, fn, radius, self.antialias)
    wx = _resample_weights(t.shape[2], ow, sx, tx, fn, radius, self.antialias)
    return torch.einsum("oh,nhwc,pw->nopc", wy, t, wx)


_prim("ScaleAndTranslate", [("kernel_type", "lanczos3"), ("antialias", True)], _scale_and_translate)


# ------------------------------------------------------------------------------------------------ sparse
def _sparse_slice(self, indices, values, shape, start, size):
    idx, val = _t(indices).long(), _t(values)
    dense, lo, ext = _t(shape).long(), _t(start).long(), _t(size).long()
    hi = torch.minimum(lo + ext, dense)
    keep = ((idx >= lo) & (idx < hi)).all(1)
    return idx[keep] - lo, val[keep], (hi - lo).clamp(min=0)


_prim("SparseSlice", (), _sparse_slice)


def identity(x):
    """Returns a tensor with the contents of ``x`` (ops/operations/other_ops.py identity)."""
    return _w(_t(x).clone())


__all__.append("identity")
