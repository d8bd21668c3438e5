"""Multi-GPU partitioning of the path: one process per GPU over torch.distributed.

The reference has no multi-GPU quantization path; the path shards naturally in two
places and this module holds the host logic for both:

* tokens: every rank accumulates H and C over its share of the calibration sequences;
  ``reduce_moments`` turns the per-rank running means into the global ones with one
  all-reduce per matrix (weights n_r / N);
* weight rows: given the (replicated) inverse-Hessian factor, rows of a layer are
  independent, so each rank corrects and quantizes a slab of rows and the slabs are
  all-gathered.  Slabs start on multiples of 32 rows so that no packed zero-point word
  straddles two ranks for any bit width.

The collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def row_slab(out_features: int, rank: int, world: int, align: int = 32):
    """[first, last) rows of ``rank``: contiguous, aligned, sizes differing by at most
    one aligned unit; trailing ranks may be empty for small layers."""
    units = (out_features + align - 1) // align
    base, extra = divmod(units, world)
    first_u = rank * base + min(rank, extra)
    last_u = first_u + base + (1 if rank < extra else 0)
    return min(first_u * align, out_features), min(last_u * align, out_features)


def seq_shard(n_seq: int, rank: int, world: int):
    """[first, last) calibration sequences of ``rank``."""
    base, extra = divmod(n_seq, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


class ShardedContext:
    """Token- and row-sharding over a process group."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._totals = {}
        self._pending_cross = None

    # ---- tokens -------------------------------------------------------------------
    def reduce_moments(self, h: torch.Tensor, c: Optional[torch.Tensor], n: int, fixed_split: bool = False,
                       defer_cross: bool = False):
        """Per-rank means (2/n_r)·Σ_r → global means (2/N)·Σ.  Returns (h, c, N).

        ``fixed_split``: the caller's token split over the ranks does not change between calls with
        the same local count (the calibration sequences of a run), so the global count is
        exchanged once and remembered, which saves a host synchronisation per call.
        ``defer_cross``: the reduction of ``c`` is only started; the caller runs what needs ``h``
        alone (the factorisation) and calls ``wait_cross()`` before it reads ``c``."""
        big_n = self._totals.get(n) if fixed_split else None
        if big_n is None:
            total = torch.tensor([float(n)], dtype=torch.float64, device=h.device)
            dist.all_reduce(total, group=self.group)
            big_n = int(total.item())
            if fixed_split:
                self._totals[n] = big_n
        w = (n / big_n) if big_n > 0 else 0.0
        h.mul_(w)
        dist.all_reduce(h, group=self.group)
        if c is not None:
            c.mul_(w)
            if defer_cross:
                self.wait_cross()
                self._pending_cross = (dist.all_reduce(c, group=self.group, async_op=True), c)
            else:
                dist.all_reduce(c, group=self.group)
        return h, c, big_n

    def wait_cross(self):
        """Make the current stream wait for a cross term whose reduction ``reduce_moments`` started."""
        pending, self._pending_cross = self._pending_cross, None
        if pending is not None:
            pending[0].wait()

    # ---- rows ---------------------------------------------------------------------
    def gather_rows(self, local: torch.Tensor, out_features: int, dim: int, per_row: float = 1.0,
                    align: int = 32) -> torch.Tensor:
        """Concatenate every rank's slab along ``dim``.  ``per_row`` is the number of
        entries along ``dim`` per weight row (bits/32 for packed zero points)."""
        sizes = []
        for r in range(self.world):
            a, b = row_slab(out_features, r, self.world, align)
            sizes.append(int(round((b - a) * per_row)))
        biggest = max(sizes)
        if biggest == 0:
            return local
        shape = list(local.shape)
        shape[dim] = biggest
        padded = torch.zeros(shape, dtype=local.dtype, device=local.device)
        padded.narrow(dim, 0, local.shape[dim]).copy_(local)
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded.contiguous(), group=self.group)
        return torch.cat([p.narrow(dim, 0, s) for p, s in zip(parts, sizes)], dim=dim)

    def gather_column_slabs(self, slabs):
        """Several 2-D results whose columns are split evenly over the ranks ([R_i, cols_i] here,
        [R_i, cols_i * world] assembled), moved by ONE all-gather of their bytes instead of one
        collective (and its padding, list and concatenation) each.  Returns the assembled tensors."""
        flat = torch.cat([t.contiguous().reshape(-1).view(torch.uint8) for t in slabs])
        everyone = torch.empty(self.world * flat.numel(), dtype=torch.uint8, device=flat.device)
        dist.all_gather_into_tensor(everyone, flat, group=self.group)
        everyone = everyone.view(self.world, flat.numel())
        out, off = [], 0
        for t in slabs:
            nbytes = t.numel() * t.element_size()
            part = everyone[:, off:off + nbytes].contiguous().view(t.dtype)
            out.append(part.reshape(self.world, t.shape[0], t.shape[1]).permute(1, 0, 2)
                       .reshape(t.shape[0], self.world * t.shape[1]))
            off += nbytes
        return out

    def quantize_rows(self, quantizer, module, h, c, cfg, factor,
                      compute: Optional[Callable] = None):
        """Correct and quantize this rank's row slab of ``module`` and assemble the full
        GPTQResult on every rank (``quantizer.results[name]``).

        ``compute(weight_slab, c) -> dict`` produces the slab's outputs (qweight
        [in·bits/32, rows], qzeros [G, rows·bits/32], scales [G, rows], zeros [G, rows],
        dequantized [rows, in]); the default runs the CUDA kernels."""
        return self.quantize_rows_stacked(quantizer, [module], h, c, cfg, factor, compute)[module]

    def quantize_rows_stacked(self, quantizer, modules, h, c, cfg, factor,
                              compute: Optional[Callable] = None):
        """``quantize_rows`` for several layers that share the Hessian and the settings: their
        weights are stacked row-wise, the stacked rows are split over the ranks, and the gathered
        result is cut back into one GPTQResult per layer (rows never interact, so the results are
        those of the per-layer calls).  Returns {module: GPTQResult}."""
        import time

        from . import kernels
        from .quantizer.gptq._gptq import GPTQ, GPTQResult

        names = [quantizer.module_to_name[m] for m in modules]
        on_gpu = modules[0].weight.is_cuda
        timer = kernels.LayerTimer(modules[0].weight.device) if on_gpu else time.time()
        bits = GPTQ.resolve_bits(names[0], quantizer.wbits, quantizer.mlp_wbits, quantizer.module_wbits)
        gs = GPTQ.resolve_groupsize(names[0], quantizer.groupsize, quantizer.mlp_groupsize)
        rows = [m.weight.shape[0] for m in modules]
        weight = modules[0].weight.data if len(modules) == 1 else torch.cat([m.weight.data for m in modules], 0)
        out_features, d = weight.shape
        first, last = row_slab(out_features, self.rank, self.world)
        slab = weight[first:last]

        default_compute = compute is None
        # results are packed exactly when the quantizer packs on one GPU
        want_packed = bool(getattr(quantizer, "bitpack_on_quantize", True))
        if compute is None:
            from .quantizer._quantizer import qep_factor

            def compute(w_slab, cross, w_hat_out=None):
                if w_slab.shape[0] == 0:
                    groups = 1 if gs == -1 else (d + gs - 1) // gs
                    dev = w_slab.device
                    empty = {
                        "scales": torch.empty((groups, 0), dtype=torch.float16, device=dev),
                        "zeros": torch.empty((groups, 0), dtype=torch.int32, device=dev),
                        "dequantized": torch.empty((0, d), dtype=w_slab.dtype, device=dev),
                    }
                    if want_packed:
                        empty["qweight"] = torch.empty((d * bits // 32, 0), dtype=torch.int32, device=dev)
                        empty["qzeros"] = torch.empty((groups, 0), dtype=torch.int32, device=dev)
                    else:
                        empty["codes"] = torch.empty((0, d), dtype=torch.int32, device=dev)
                    return empty
                if cross is not None:
                    # the correction has its own damping and retry rule: reuse the column loop's
                    # factor only where one GPU would (same bytes on every rank either way)
                    kernels.qep_adjust(w_slab, cross, qep_factor(h, factor, cfg.percdamp), cfg.perccorr)
                outputs = {"dequantized": w_hat_out} if w_hat_out is not None else None
                return kernels.gptq_quantize(w_slab, factor, wbits=bits, groupsize=gs, sym=quantizer.sym,
                                             blocksize=quantizer.blocksize, pack=want_packed,
                                             want_codes=not want_packed, outputs=outputs,
                                             mse=bool(quantizer.mse), q_grid=quantizer.q_grid,
                                             q_norm=quantizer.q_norm)

        # Equal slabs on NCCL: the column loop writes this rank's rows of the propagated weight
        # straight into its place in the all-gather buffer and the gather runs in place.
        w_full = None
        if (default_compute and weight.is_cuda and dist.get_backend(self.group) == "nccl"
                and out_features % (32 * self.world) == 0):
            w_full = torch.empty((out_features, d), dtype=weight.dtype, device=weight.device)
            local = compute(slab, c, w_full[first:last])
            dist.all_gather_into_tensor(w_full, w_full[first:last], group=self.group)
            w_hat = w_full
        else:
            local = compute(slab, c)
            w_hat = self.gather_rows(local["dequantized"], out_features, dim=0)
        packed = "qweight" in local
        if packed and out_features % (32 * self.world) == 0:
            # equal slabs: the three column-split results travel in one collective
            qweight, qzeros, scales = self.gather_column_slabs(
                [local["qweight"], local["qzeros"], local["scales"]])
        elif packed:
            qweight = self.gather_rows(local["qweight"], out_features, dim=1)
            qzeros = self.gather_rows(local["qzeros"], out_features, dim=1, per_row=bits / 32.0)
        else:
            # bit widths without a packed layout (or bitpack_on_quantize=False): integer codes
            # [rows, in] and raw zero points [G, rows], as on one GPU
            qweight = self.gather_rows(local["codes"], out_features, dim=0)
            qzeros = self.gather_rows(local["zeros"], out_features, dim=1)
        if not (packed and out_features % (32 * self.world) == 0):
            scales = self.gather_rows(local["scales"], out_features, dim=1)
        perm = getattr(factor, "perm", None) if quantizer.actorder else None
        pieces, r0 = [], 0
        for r in rows:
            if packed:
                pieces += [qweight[:, r0:r0 + r], scales[:, r0:r0 + r],
                           qzeros[:, r0 * bits // 32:(r0 + r) * bits // 32]]
            else:
                pieces += [qweight[r0:r0 + r], scales[:, r0:r0 + r], qzeros[:, r0:r0 + r]]
            r0 += r
        perm64 = perm.to(torch.int64) if perm is not None else None
        if qweight.is_cuda:
            host = kernels.to_host(pieces + [perm64] * len(rows))   # may still be in flight: not read here
        else:
            host = [p.contiguous() for p in pieces] + [perm64.clone() if perm64 is not None else None
                                                       for _ in rows]
        results, r0 = {}, 0
        for i, (m, name, r) in enumerate(zip(modules, names, rows)):
            qw, sc, qz = host[3 * i], host[3 * i + 1], host[3 * i + 2]
            if gs == -1 and not packed:
                qz = qz.reshape(r, 1)
            result = GPTQResult(
                wbits=bits, groupsize=gs, actorder=quantizer.actorder, sym=quantizer.sym,
                qweight=qw, scales=(sc if gs != -1 else sc.reshape(r, 1)), qzeros=qz,
                perm=host[3 * len(rows) + i],
                qweight_is_packed=packed, qzeros_is_packed=packed, qweight_original_shape=(r, d),
            )
            result.__dict__["_device_dequantized"] = w_hat[r0:r0 + r]
            quantizer.results[name] = result
            results[m] = result
            r0 += r
        if on_gpu:
            timer.stop([(results[m], r / out_features) for m, r in zip(modules, rows)])
        else:
            for m, r in zip(modules, rows):
                results[m].quantization_time = (time.time() - timer) * r / out_features
        return results

    # ---- independent layers (MoE experts) ---------------------------------------------
    def quantize_independent(self, quantizer, items, compute: Optional[Callable] = None):
        """Layers with a Hessian of their own (experts of a mixture, each calibrated on the tokens
        routed to it) are independent problems: they are dealt round-robin to the ranks, each rank
        factors and quantizes its layers whole, and the results are broadcast from their owners so
        that every rank holds every GPTQResult and every propagated weight.

        ``items``: list of (module, hessian) with the Hessian already reduced over the ranks, in the
        same order on every rank.  ``compute(weight, hessian) -> dict`` (qweight, qzeros, scales,
        dequantized, optionally perm) replaces the CUDA kernels in CPU tests.
        Returns {module: GPTQResult}; ``quantizer.results`` is filled as well."""
        import time

        from . import kernels
        from .quantizer.gptq._gptq import GPTQ, GPTQResult

        results = {}
        local = {}
        t_local = {}
        mine = [(i, item) for i, item in enumerate(items) if i % self.world == self.rank]
        if compute is None:
            # this rank's layers, several at a time on separate streams
            outs = quantizer.independent_on_device([item for _i, item in mine])
            for (i, _item), out in zip(mine, outs):
                local[i], t_local[i] = out, out["seconds"]
        else:
            for i, (module, hessian) in mine:
                t0 = time.time()
                local[i] = compute(module.weight.data, hessian)
                t_local[i] = time.time() - t0
        for i, (module, _h) in enumerate(items):
            owner = i % self.world
            name = quantizer.module_to_name[module]
            bits = GPTQ.resolve_bits(name, quantizer.wbits, quantizer.mlp_wbits, quantizer.module_wbits)
            gs = GPTQ.resolve_groupsize(name, quantizer.groupsize, quantizer.mlp_groupsize)
            out_features, d = module.weight.shape
            groups = 1 if gs == -1 else (d + gs - 1) // gs
            dev = module.weight.device
            shapes = {
                "qweight": ((d * bits // 32, out_features), torch.int32),
                "qzeros": ((groups, out_features * bits // 32), torch.int32),
                "scales": ((groups, out_features), torch.float16),
                "dequantized": ((out_features, d), module.weight.dtype),
            }
            if quantizer.actorder:
                shapes["perm"] = ((d,), torch.int64)
            got = {}
            for key, (shape, dtype) in shapes.items():
                if owner == self.rank:
                    buf = local[i][key].to(device=dev, dtype=dtype).contiguous()
                else:
                    buf = torch.empty(shape, dtype=dtype, device=dev)
                dist.broadcast(buf, src=dist.get_global_rank(self.group, owner) if self.group is not None else owner,
                               group=self.group)
                got[key] = buf
            elapsed = torch.tensor([t_local.get(i, 0.0)], dtype=torch.float64, device=dev)
            dist.broadcast(elapsed, src=dist.get_global_rank(self.group, owner) if self.group is not None else owner,
                           group=self.group)
            pieces = [got["qweight"], got["scales"], got["qzeros"], got.get("perm")]
            host = kernels.to_host(pieces) if dev.type == "cuda" else pieces
            result = GPTQResult(
                wbits=bits, groupsize=gs, actorder=quantizer.actorder, sym=quantizer.sym, qweight=host[0],
                scales=(host[1] if gs != -1 else host[1].reshape(out_features, 1)), qzeros=host[2], perm=host[3],
                qweight_is_packed=True, qzeros_is_packed=True, qweight_original_shape=(out_features, d),
            )
            result.__dict__["_device_dequantized"] = got["dequantized"]
            result.quantization_time = float(elapsed.item())
            quantizer.results[name] = result
            results[module] = result
            local.pop(i, None)
        return results
