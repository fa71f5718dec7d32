"""Single-box batch partitioner: one call, the batch sharded over several B200s.

The signature of every path is independent, forward and backward, so the batch is cut
into contiguous slices (remainder to the first devices), each device works on its slice
with its own streams, and nothing is exchanged between devices.  The reference has no
multi-GPU path; this module is the new layer between the Python operators and the C ABI.

Three entry points:

* ``sig_sharded`` / ``sig_backprop_sharded``: host arrays (NumPy / CPU tensors) through the
  C-side partitioner (``sigb200_signature_sharded_*``: one host thread per device, copies
  overlapped with compute); host array in, host array out.
* ``sig_multi_device``: torch tensors, differentiable.  One tensor is scattered over the
  devices with ``.to(device)`` (which autograd follows), or a list of tensors already
  resident on different devices is taken as it is; ``torch_api.sig`` runs on every shard's own
  device and stream (launches are asynchronous, so the devices work concurrently), and the
  per-device results come back as a list or, with ``gather_to``, as one tensor on one device.
* ``all_gather_signatures``: the one collective this path can have, for the one-process-per-GPU
  layout (``torch.distributed``): a single all-gather of every rank's shard of results."""
import ctypes

import numpy as np
import torch

from . import load_cusig
from .data_handlers import Output, PathInput, SigInput, check_same
from .error_codes import err_msg
from .param_checks import check_non_neg, check_type
from .sig_length import infer_scalar_term, sig_length


def shard_bounds(batch_size, n_shards):
    """[(begin, end)] of contiguous shards; the first ``batch_size % n_shards`` get one extra."""
    n = max(1, min(n_shards, max(batch_size, 1)))
    chunk, rem = divmod(batch_size, n)
    bounds, begin = [], 0
    for g in range(n):
        end = begin + chunk + (1 if g < rem else 0)
        bounds.append((begin, end))
        begin = end
    return bounds


def _device_array(devices):
    if devices is None:
        return None, torch.cuda.device_count()
    arr = (ctypes.c_int * len(devices))(*[int(d) for d in devices])
    return arr, len(devices)


def sig_sharded(path, degree, *, devices=None, time_aug=False, lead_lag=False, end_time=1., scalar_term=False):
    """``sig`` of a host-resident batch computed on several GPUs; returns a host array."""
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    data = PathInput(path, time_aug, lead_lag, end_time)
    if data.device != "cpu":
        raise ValueError("sig_sharded takes host arrays; for CUDA tensors call sig on each device's shard")
    result = Output(data, (sig_length(data.dimension, degree, scalar_term=scalar_term),))
    if data.batch_size == 0:
        return result.array
    dev, n = _device_array(devices)
    code = load_cusig.fn("sigb200_signature_sharded", data.dtype)(
        data.pointer, result.pointer, data.batch_size, data.data_dimension, data.data_length, degree,
        time_aug, lead_lag, end_time, scalar_term, dev, n)
    if code:
        raise Exception("Error in pysiglib.sig: " + err_msg(code))
    return result.array


def sig_backprop_sharded(path, sig, sig_derivs, degree, *, devices=None, time_aug=False, lead_lag=False,
                         end_time=1.):
    """``sig_backprop`` of a host-resident batch computed on several GPUs."""
    check_type(degree, "degree", int)
    check_non_neg(degree, "degree")
    data = PathInput(path, time_aug, lead_lag, end_time)
    if data.device != "cpu":
        raise ValueError("sig_backprop_sharded takes host arrays")
    infer_scalar_term(sig, data.data_dimension, degree, time_aug=time_aug, lead_lag=lead_lag)
    n_sig = sig_length(data.dimension, degree, scalar_term=False)
    sig_in, der_in = SigInput(sig, n_sig, "sig"), SigInput(sig_derivs, n_sig, "sig_derivs")
    check_same([sig_in, der_in], ["sig", "sig_derivs"])
    if data.kind != sig_in.kind or data.dtype != sig_in.dtype or data.batch_shape != sig_in.batch_shape:
        raise ValueError("path, sig and sig_derivs must agree in array type, dtype and batch shape")
    result = Output(data, (data.data_length, data.data_dimension))
    if data.batch_size == 0:
        return result.array
    dev, n = _device_array(devices)
    code = load_cusig.fn("sigb200_sig_backprop_sharded", data.dtype)(
        data.pointer, result.pointer, der_in.pointer, sig_in.pointer, data.batch_size, data.data_dimension,
        data.data_length, degree, time_aug, lead_lag, end_time, False, dev, n)
    if code:
        raise Exception("Error in pysiglib.sig_backprop: " + err_msg(code))
    return result.array


def sig_multi_device(path, degree, *, devices=None, gather_to=None, time_aug=False, lead_lag=False, end_time=1.,
                     scalar_term=False):
    """Differentiable ``sig`` of a batch spread over several GPUs of one box.

    :param path: a tensor ``(B, L, d)`` on any device (scattered over ``devices`` in contiguous
        batch slices, remainder to the first devices), or a list of tensors ``(B_g, L, d)`` that
        already live on the devices that should process them.
    :param devices: device ordinals for the scatter (default: all visible GPUs); ignored for a list.
    :param gather_to: ``None`` returns the list of per-device results; a device (``"cuda:0"``,
        ``"cpu"``, a ``torch.device``) returns their concatenation on that device.
    Gradients flow back through the gather, the per-shard ``Sig`` function and the scatter to
    wherever ``path`` lives; no collective and no cross-device reduction is involved (the
    gradient of a path depends on that path only).
    """
    from .torch_api import sig as sig_autograd
    if isinstance(path, (list, tuple)):
        shards = list(path)
        if not shards or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in shards):
            raise ValueError("a list passed to sig_multi_device must hold CUDA tensors")
    else:
        if not isinstance(path, torch.Tensor) or path.dim() != 3:
            raise ValueError("sig_multi_device takes a (batch, length, dimension) tensor or a list of CUDA tensors")
        if devices is None:
            devices = list(range(torch.cuda.device_count()))
        if not devices:
            raise ValueError("no CUDA device to shard over")
        bounds = shard_bounds(path.shape[0], len(devices))
        shards = [path[b:e].to(torch.device("cuda", int(dev))) for (b, e), dev in zip(bounds, devices) if e > b]
    results = []
    for shard in shards:
        with torch.cuda.device(shard.device):
            results.append(sig_autograd(shard, degree, time_aug=time_aug, lead_lag=lead_lag, end_time=end_time,
                                        scalar_term=scalar_term))
    if gather_to is None:
        return results
    target = torch.device(gather_to)
    return torch.cat([r.to(target) for r in results], dim=0)


def all_gather_signatures(local, batch_size=None, group=None):
    """One-process-per-GPU layout: every rank holds the signatures ``(B_rank, S)`` of its
    contiguous shard (``shard_bounds(batch_size, world_size)[rank]``); returns the ``(batch_size,
    S)`` tensor of all of them on every rank with ONE ``all_gather_into_tensor``.  Ragged shards
    (``batch_size`` not divisible by the number of ranks) are padded to the largest shard for the
    collective and trimmed afterwards."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if batch_size is None:
        batch_size = local.shape[0] * world
    bounds = shard_bounds(batch_size, world)
    biggest = max(e - b for b, e in bounds)
    if local.shape[0] != bounds[dist.get_rank(group)][1] - bounds[dist.get_rank(group)][0]:
        raise ValueError("this rank's shard has %d rows, expected %d" % (
            local.shape[0], bounds[dist.get_rank(group)][1] - bounds[dist.get_rank(group)][0]))
    send = local
    if local.shape[0] != biggest:
        send = local.new_zeros((biggest,) + tuple(local.shape[1:]))
        send[: local.shape[0]] = local
    out = local.new_empty((world * biggest,) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, send.contiguous(), group=group)
    if all(e - b == biggest for b, e in bounds):
        return out
    return torch.cat([out[g * biggest: g * biggest + (e - b)] for g, (b, e) in enumerate(bounds)], dim=0)
