"""Layer-stack driver over the C ABI: runs a list of sparse convolutions
(workloads.Layer) the way a framework plugin would call the library.

Per distinct geometry one mluOpGetIndicePairs call (layers that share a
`rulebook` name share its result) whose indice_num output is pinned host memory
(mluOpIndiceConvolutionForward takes the counts as a host array), then per layer
one mluOpIndiceConvolutionForward call.  All work is enqueued on the handle's stream.

The driver keeps its descriptors and its pinned host buffer alive between steps
and re-sets only the dimensions that change, so that the host side adds as little
as possible to the gaps the API's two host round trips per rulebook leave on the
GPU.
"""
import contextlib
import ctypes
import sys
import time

import torch

# The package directory name is not a Python identifier, so the package is
# loaded by path under the name "mluops_b200" (see __graft_entry__.load_package);
# this module is always imported as its submodule.
ops = sys.modules[__package__]

_vp = ctypes.c_void_p


class Workspace:
    """One device scratch buffer, grown on demand and reused by every call."""

    def __init__(self, device):
        self.device = device
        self.buf = torch.empty((1,), dtype=torch.uint8, device=device)

    def get(self, nbytes):
        if self.buf.numel() < nbytes:
            self.buf = torch.empty((int(nbytes * 1.25) + 256,), dtype=torch.uint8, device=self.device)
        return self.buf


class LayerRecord:
    """What one layer consumed and produced (kept for parity checks and roofline accounting)."""
    __slots__ = ("layer", "n_in", "n_out", "indice_num", "pairs", "in_indices", "out_indices", "features_in",
                 "features_out", "new_rulebook", "in_space", "out_space", "weights", "rulebook")


class Rulebook:
    """Outputs of one mluOpGetIndicePairs call as the driver keeps them."""
    __slots__ = ("pairs", "out_indices", "indice_num", "n_out", "table", "in_space", "out_space", "in_indices",
                 "input_table")


class RulebookPlan:
    """All rulebooks of one batch (plan_rulebooks) for run_convolutions."""

    def __init__(self):
        self.rulebooks = {}
        self.out_indices = None
        self.reuse_tables = False
        self.done = None


class _Desc:
    """A tensor descriptor that lives as long as the driver; dims are re-set per call."""

    def __init__(self, layout, dtype):
        self.layout, self.dtype = layout, dtype
        self.ptr = _vp()
        ops.check("mluOpCreateTensorDescriptor", ops.lib().mluOpCreateTensorDescriptor(ctypes.byref(self.ptr)))

    def set(self, *dims):
        arr = (ctypes.c_int64 * len(dims))(*dims)
        ops.check("mluOpSetTensorDescriptor_v2",
                  ops.lib().mluOpSetTensorDescriptor_v2(self.ptr, self.layout, self.dtype, len(dims), arr))
        return self.ptr

    def destroy(self):
        if self.ptr:
            ops.lib().mluOpDestroyTensorDescriptor(self.ptr)
            self.ptr = _vp()


class SparseNetwork:
    def __init__(self, handle, layers, weights, grid, batch, rulebook_handle=None, rulebook_stream=None):
        """weights: per layer a CUDA tensor in ARRAY layout [kd,kh,kw,Ci,Co].

        rulebook_handle / rulebook_stream: a second library handle bound to a second
        (torch) stream.  Rulebooks depend only on coordinates, never on features, so with
        them mluOpGetIndicePairs runs on that stream and the host waits there, while the
        convolutions already enqueued on the first handle's stream keep the GPU busy."""
        self.handle, self.layers, self.weights = handle, layers, weights
        self.rulebook_handle, self.rulebook_stream = rulebook_handle, rulebook_stream
        self.grid, self.batch = list(grid), int(batch)
        dev = weights[0].device
        self.device = dev
        self.workspace = Workspace(dev)
        self.rulebook_workspace = Workspace(dev) if rulebook_handle is not None else None
        self.lib = ops.lib()
        ft = ops.DTYPE_HALF if weights[0].dtype == torch.float16 else ops.DTYPE_FLOAT
        self.d_idx = _Desc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32)
        self.d_pairs = _Desc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32)
        self.d_out_idx = _Desc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32)
        self.d_num = _Desc(ops.LAYOUT_ARRAY, ops.DTYPE_INT32)
        self.d_feat = _Desc(ops.LAYOUT_ARRAY, ft)
        self.d_fout = _Desc(ops.LAYOUT_ARRAY, ft)
        self.d_filt = []
        for w in weights:
            d = _Desc(ops.LAYOUT_ARRAY, ft)
            d.set(*w.shape)
            self.d_filt.append(d)
        # geometry per rulebook name: the spaces are fixed by the grid and the layer list
        self.geometry = {}
        space = list(self.grid)
        for ly in layers:
            if ly.rulebook not in self.geometry:
                out_space = list(space) if ly.sub_m else ops.output_space(space, ly.pad, ly.stride, ly.dilation,
                                                                           ly.filter_space)
                conv = ops.SparseConvDesc(self.batch, ly.pad, ly.stride, ly.dilation, space, ly.filter_space,
                                          out_space, ly.sub_m)
                self.geometry[ly.rulebook] = (conv, list(space), out_space)
            if not ly.sub_m:
                space = self.geometry[ly.rulebook][2]
        max_k = max(ly.kernel_volume for ly in layers)
        # one pinned row of counts per rulebook, so that a count that is read late is still there
        self.num_slot = {name: i for i, name in enumerate(self.geometry)}
        self.num_host = torch.empty((len(self.geometry), max_k), dtype=torch.int32).pin_memory()
        self.zero_i64 = (ctypes.c_int64 * max_k)()
        self.num_i64 = (ctypes.c_int64 * max_k)()
        self.n_act = ctypes.c_int(0)
        self.size = ctypes.c_size_t(0)
        # {"rulebook_wait_s": host seconds spent waiting for rulebook counts, "steps": n}, or None (no timing)
        self.timers = None

    def close(self):
        for d in [self.d_idx, self.d_pairs, self.d_out_idx, self.d_num, self.d_feat, self.d_fout] + self.d_filt:
            d.destroy()
        for conv, _, _ in self.geometry.values():
            conv.destroy()

    def forward(self, indices, features, keep=False, on_final_indices=None, on_host_idle=None, reuse_tables=False,
                defer_counts=False):
        """indices [L,4] int32, features [L,Cin] on the GPU.
        Returns (features_out, out_indices, records).

        on_final_indices(out_indices, ready_event), if given, is called once, as soon as
        the coordinates of the final rows are known (when the last layer's rulebook has
        been generated) and after that layer's convolution has been enqueued, so that a
        caller can ship them while the remaining convolutions run; ready_event marks the
        point of the stream after which the rows are valid.

        on_host_idle(layer_index), if given, is called before every rulebook generation:
        the convolutions enqueued since the previous rulebook are still running and the
        host is about to wait for the rulebook's counts, so host work done here (e.g.
        enqueuing a collective for the previous step's rows) costs no GPU time.

        reuse_tables: build the neighbour table of a rulebook once
        (mluOpBuildIndiceNeighbourTable) and run its convolutions through
        mluOpIndiceConvolutionForwardFromTable, instead of the reference-shaped
        mluOpIndiceConvolutionForward that rebuilds the table in every call.

        defer_counts (with reuse_tables): a submanifold rulebook that emits its own table needs
        nothing from the host before its convolutions can be enqueued (the active outputs are the
        inputs, the table is on the device), so the host does not wait for it: the convolutions
        are ordered after it on the device, its records carry indice_num = None, and
        resolve_counts(records) fills them in after the step."""
        second = self.rulebook_handle is not None
        compute = torch.cuda.current_stream()
        if second:
            # the coordinates are ready where the caller's stream is now
            self.rulebook_stream.wait_stream(compute)
        final_rulebook = self.layers[-1].rulebook
        ready = None
        rulebooks = {}
        records = []
        cur_idx, cur_feat = indices, features
        for li, (ly, w) in enumerate(zip(self.layers, self.weights)):
            new_rb = ly.rulebook not in rulebooks
            if new_rb:
                if on_host_idle is not None:
                    on_host_idle(li)
                rulebooks[ly.rulebook] = self._generate_rulebook(ly, cur_idx, compute, reuse_tables, defer_counts)
                if on_final_indices is not None and ly.rulebook == final_rulebook:
                    ready = torch.cuda.Event()
                    ready.record(self.rulebook_stream if second else compute)
            rb = rulebooks[ly.rulebook]
            out = self._convolve(li, ly, w, cur_feat, rb, reuse_tables)
            records.append(self._record(ly, cur_feat, out, cur_idx, rb, new_rb, keep))
            cur_feat = out
            if not ly.sub_m:
                cur_idx = rb.out_indices[:rb.n_out]
            if ready is not None:
                on_final_indices(cur_idx, ready)
                ready = None
        return cur_feat, cur_idx, records

    def plan_rulebooks(self, indices, ready=None, reuse_tables=False):
        """Every rulebook of the layer list from the input coordinates alone (rulebooks never
        depend on features), on the rulebook stream when the driver has one; the host waits
        there for the counts the API hands back.  `ready` (a CUDA event, optional) marks the
        point after which `indices` is valid; without it the caller guarantees that it already
        is.  Returns a plan for run_convolutions().  A serving loop calls this for batch i+1
        right after it has enqueued run_convolutions() of batch i, so that the rulebook
        kernels and the host waits of one batch overlap the convolutions of the one before."""
        second = self.rulebook_handle is not None
        compute = torch.cuda.current_stream()
        if ready is not None:
            (self.rulebook_stream if second else compute).wait_event(ready)
        plan = RulebookPlan()
        cur_idx = indices
        for ly in self.layers:
            if ly.rulebook not in plan.rulebooks:
                rb = self._generate_rulebook(ly, cur_idx, compute, reuse_tables, False, record_for=None)
                rb.in_indices = cur_idx
                plan.rulebooks[ly.rulebook] = rb
            if not ly.sub_m:
                rb = plan.rulebooks[ly.rulebook]
                cur_idx = rb.out_indices[:rb.n_out]
        plan.out_indices = cur_idx
        plan.reuse_tables = reuse_tables
        plan.done = torch.cuda.Event()
        plan.done.record(self.rulebook_stream if second else compute)
        return plan

    def run_convolutions(self, plan, features, keep=False):
        """The convolutions of the layer list on the current stream, from a plan of
        plan_rulebooks(); nothing here waits on the host.  Returns (features_out, out_indices,
        records)."""
        compute = torch.cuda.current_stream()
        compute.wait_event(plan.done)
        records, seen = [], set()
        cur_feat = features
        for li, (ly, w) in enumerate(zip(self.layers, self.weights)):
            rb = plan.rulebooks[ly.rulebook]
            for t in (rb.pairs, rb.out_indices, rb.table):
                if t is not None and self.rulebook_handle is not None:
                    t.record_stream(compute)
            out = self._convolve(li, ly, w, cur_feat, rb, plan.reuse_tables)
            records.append(self._record(ly, cur_feat, out, rb.in_indices, rb, ly.rulebook not in seen, keep))
            seen.add(ly.rulebook)
            cur_feat = out
        return cur_feat, plan.out_indices, records

    def _generate_rulebook(self, ly, cur_idx, compute, reuse_tables, defer_counts, record_for="compute"):
        """One mluOpGetIndicePairs call (or its table-emitting extension) and the host read of
        its counts.  record_for="compute": the outputs, allocated on the rulebook stream, are
        marked as used by `compute` right away (forward()); None: the caller does that."""
        lib, h = self.lib, self.handle.ptr
        second = self.rulebook_handle is not None
        hr = self.rulebook_handle.ptr if second else h
        conv, in_space, out_space = self.geometry[ly.rulebook]
        K = ly.kernel_volume
        L = cur_idx.shape[0]
        out_rows = L if ly.sub_m else ops.max_active_outputs(L, self.batch, out_space, ly.filter_space, ly.stride,
                                                             ly.dilation)
        d_in, d_pairs = self.d_idx.set(L, 4), self.d_pairs.set(K, 2, L)
        d_out, d_num = self.d_out_idx.set(out_rows, 4), self.d_num.set(K)
        table = None
        slot = self.num_host[self.num_slot[ly.rulebook]]
        with (torch.cuda.stream(self.rulebook_stream) if second else contextlib.nullcontext()):
            pairs = torch.empty((K, 2, L), dtype=torch.int32, device=self.device)
            out_idx = torch.empty((out_rows, 4), dtype=torch.int32, device=self.device)
            ops.check("mluOpGetIndicePairsWorkspaceSize",
                      lib.mluOpGetIndicePairsWorkspaceSize(hr, conv.ptr, d_in, d_pairs, d_out, d_num,
                                                           ctypes.byref(self.size)))
            ws_bytes = self.size.value
            ws = (self.rulebook_workspace if second else self.workspace).get(ws_bytes)
            args = [hr, conv.ptr, d_in, _vp(cur_idx.data_ptr()), _vp(ws.data_ptr()), ws_bytes, d_pairs,
                    _vp(pairs.data_ptr()), d_out, _vp(out_idx.data_ptr()), d_num, _vp(slot.data_ptr())]
            if reuse_tables and ly.sub_m:
                # submanifold rulebooks leave their neighbour table behind themselves
                ops.check("mluOpGetIndiceNeighbourTableSize",
                          lib.mluOpGetIndiceNeighbourTableSize(hr, d_pairs, L, ctypes.byref(self.size)))
                table = torch.empty((max(self.size.value, 16),), dtype=torch.uint8, device=self.device)
                st = lib.mluOpGetIndicePairsWithNeighbourTable(*args, _vp(table.data_ptr()), table.numel())
                if st == ops.STATUS_NOT_SUPPORTED:
                    table = None
                else:
                    ops.check("mluOpGetIndicePairsWithNeighbourTable", st)
            if table is None:
                ops.check("mluOpGetIndicePairs", lib.mluOpGetIndicePairs(*args))
            deferred = defer_counts and table is not None
            if deferred:
                if second:  # order the convolutions after the rulebook on the device
                    done = torch.cuda.Event()
                    done.record(self.rulebook_stream)
                    compute.wait_event(done)
            else:
                # The convolution API takes indice_num as a host array, so the rulebook writes it
                # straight into pinned host memory (device-accessible under unified addressing):
                # no copy is queued on the copy engines, only the rulebook's stream has to drain.
                if self.timers is not None:
                    t_wait = time.perf_counter()
                torch.cuda.current_stream().synchronize()
                if self.timers is not None:
                    self.timers["rulebook_wait_s"] = self.timers.get("rulebook_wait_s", 0.0) + \
                        time.perf_counter() - t_wait
        lib.mluOpGetSparseConvolutionNumActOut(conv.ptr, ctypes.byref(self.n_act))
        n_out = self.n_act.value
        num_list = None if deferred else slot[:K].tolist()
        if reuse_tables and table is None:
            # (built on the convolutions' stream, where the rulebook is complete: the host has waited for it)
            for i, v in enumerate(num_list):
                self.num_i64[i] = v
            with (torch.cuda.stream(self.rulebook_stream) if second and record_for is None
                  else contextlib.nullcontext()):
                ops.check("mluOpGetIndiceNeighbourTableSize",
                          lib.mluOpGetIndiceNeighbourTableSize(h, d_pairs, n_out, ctypes.byref(self.size)))
                table = torch.empty((max(self.size.value, 16),), dtype=torch.uint8, device=self.device)
                ops.check("mluOpBuildIndiceNeighbourTable",
                          lib.mluOpBuildIndiceNeighbourTable(hr if second and record_for is None else h, d_pairs,
                                                             _vp(pairs.data_ptr()), self.num_i64, n_out,
                                                             _vp(table.data_ptr()), table.numel()))
        if second and record_for == "compute":
            # allocated on the rulebook stream, read by the convolutions on the other one
            for t in (pairs, out_idx, table):
                if t is not None:
                    t.record_stream(compute)
        rb = Rulebook()
        rb.pairs, rb.out_indices, rb.indice_num, rb.n_out, rb.table = pairs, out_idx, num_list, n_out, table
        rb.in_space, rb.out_space, rb.in_indices = list(in_space), list(out_space), cur_idx
        return rb

    def _convolve(self, li, ly, w, cur_feat, rb, reuse_tables):
        """One mluOpIndiceConvolutionForward call (or its from-table extension) on the current stream."""
        lib, h = self.lib, self.handle.ptr
        K, L, n_out = ly.kernel_volume, cur_feat.shape[0], rb.n_out
        # (a convolution from a table reads the pairs from the table: the counts it is handed
        # only size its trace accounting, so a rulebook that was not waited for passes zeros)
        for i, v in enumerate(rb.indice_num if rb.indice_num is not None else self.zero_i64[:K]):
            self.num_i64[i] = v
        out = torch.empty((n_out, ly.co), dtype=cur_feat.dtype, device=self.device)
        d_f, d_p, d_o = self.d_feat.set(L, ly.ci), self.d_pairs.set(K, 2, L), self.d_fout.set(n_out, ly.co)
        d_w = self.d_filt[li].ptr
        table = rb.table if reuse_tables else None
        if table is not None:
            ops.check("mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize",
                      lib.mluOpGetIndiceConvolutionForwardFromTableWorkspaceSize(
                          h, d_f, d_w, d_p, d_o, self.num_i64, n_out, 0, ly.sub_m, ctypes.byref(self.size)))
            ws = self.workspace.get(self.size.value)
            ops.check("mluOpIndiceConvolutionForwardFromTable",
                      lib.mluOpIndiceConvolutionForwardFromTable(
                          h, d_f, _vp(cur_feat.data_ptr()), d_w, _vp(w.data_ptr()), d_p, _vp(table.data_ptr()),
                          table.numel(), self.num_i64, n_out, 0, ly.sub_m, _vp(ws.data_ptr()), self.size.value,
                          d_o, _vp(out.data_ptr())))
        else:
            ops.check("mluOpGetIndiceConvolutionForwardWorkspaceSize",
                      lib.mluOpGetIndiceConvolutionForwardWorkspaceSize(h, d_f, d_w, d_p, d_o, self.num_i64, n_out, 0,
                                                                        ly.sub_m, ctypes.byref(self.size)))
            ws = self.workspace.get(self.size.value)
            ops.check("mluOpIndiceConvolutionForward",
                      lib.mluOpIndiceConvolutionForward(h, d_f, _vp(cur_feat.data_ptr()), d_w, _vp(w.data_ptr()), d_p,
                                                        _vp(rb.pairs.data_ptr()), self.num_i64, n_out, 0, ly.sub_m,
                                                        _vp(ws.data_ptr()), self.size.value, d_o,
                                                        _vp(out.data_ptr())))
        return out

    def _record(self, ly, features_in, features_out, in_indices, rb, new_rb, keep):
        rec = LayerRecord()
        rec.layer, rec.n_in, rec.n_out = ly, features_in.shape[0], rb.n_out
        rec.indice_num, rec.new_rulebook = rb.indice_num, new_rb
        if keep:
            rec.rulebook = rb
            rec.pairs, rec.in_indices, rec.out_indices = rb.pairs, in_indices, rb.out_indices[:rb.n_out]
            rec.features_in, rec.features_out = features_in, features_out
            rec.in_space, rec.out_space = list(rb.in_space), list(rb.out_space)
        return rec

    def resolve_counts(self, records):
        """Fills in the pair counts of records whose rulebook was not waited for (defer_counts);
        waits for the device first."""
        torch.cuda.synchronize(self.device)
        for rec in records:
            if rec.indice_num is None:
                K = rec.layer.kernel_volume
                rec.indice_num = self.num_host[self.num_slot[rec.layer.rulebook], :K].tolist()
        return records

    def backward(self, records, grad_out, reuse_tables=False):
        """Gradients of the layer stack, last layer first, from the records of
        forward(keep=True) and the gradient of its final features.  Per layer one
        mluOpIndiceConvolutionBackwardFilter and one mluOpIndiceConvolutionBackwardData
        call on the rulebook the forward pass generated.  reuse_tables: one input
        neighbour table per rulebook (mluOpBuildIndiceInputNeighbourTable) feeds the input
        gradients of all its layers (...BackwardDataFromTable), and the filter gradients take
        the forward table the rulebook kept (forward(reuse_tables=True)) where their kernel
        works from one (...BackwardFilterFromTable).  Returns (input_grad of the first layer,
        [filters_grad per layer])."""
        lib, h = self.lib, self.handle.ptr
        grad = grad_out
        filter_grads = [None] * len(records)
        for li in range(len(records) - 1, -1, -1):
            rec, w = records[li], self.weights[li]
            ly = rec.layer
            K, L, n_out = ly.kernel_volume, rec.n_in, rec.n_out
            for i, v in enumerate(rec.indice_num):
                self.num_i64[i] = v
            d_f, d_g = self.d_feat.set(L, ly.ci), self.d_fout.set(n_out, ly.co)
            d_p, d_w = self.d_pairs.set(K, 2, L), self.d_filt[li].ptr
            dw = torch.empty_like(w)
            ops.check("mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize",
                      lib.mluOpGetIndiceConvolutionBackwardFilterWorkspaceSize(h, d_f, d_g, d_p, d_w, self.num_i64, 0,
                                                                               ly.sub_m, ctypes.byref(self.size)))
            ws = self.workspace.get(self.size.value)
            rb = rec.rulebook
            st = ops.STATUS_NOT_SUPPORTED
            if reuse_tables and getattr(rb, "table", None) is not None:
                st = lib.mluOpIndiceConvolutionBackwardFilterFromTable(
                    h, d_f, _vp(rec.features_in.data_ptr()), d_g, _vp(grad.data_ptr()), d_p, _vp(rb.table.data_ptr()),
                    rb.table.numel() * 4, self.num_i64, 0, ly.sub_m, _vp(ws.data_ptr()), self.size.value, d_w,
                    _vp(dw.data_ptr()))
                if st != ops.STATUS_NOT_SUPPORTED:
                    ops.check("mluOpIndiceConvolutionBackwardFilterFromTable", st)
            if st == ops.STATUS_NOT_SUPPORTED:
                ops.check("mluOpIndiceConvolutionBackwardFilter",
                          lib.mluOpIndiceConvolutionBackwardFilter(h, d_f, _vp(rec.features_in.data_ptr()), d_g,
                                                                   _vp(grad.data_ptr()), d_p,
                                                                   _vp(rec.pairs.data_ptr()), self.num_i64, 0,
                                                                   ly.sub_m, _vp(ws.data_ptr()), self.size.value,
                                                                   d_w, _vp(dw.data_ptr())))
            filter_grads[li] = dw
            dx = torch.empty((L, ly.ci), dtype=grad.dtype, device=self.device)
            centred = ly.sub_m and all(s == 1 for s in ly.stride) and all(d == 1 for d in ly.dilation) and all(
                k % 2 == 1 and p == k // 2 for k, p in zip(ly.filter_space, ly.pad))
            if reuse_tables and K <= 128 and centred and getattr(rb, "table", None) is not None:
                # a centred submanifold rulebook is symmetric: its forward table, offsets mirrored, is its
                # input table (where the tensor-memory kernel runs; NOT_SUPPORTED otherwise)
                ops.check("mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize",
                          lib.mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(
                              h, d_g, d_w, d_p, d_f, self.num_i64, 0, ctypes.byref(self.size)))
                ws = self.workspace.get(self.size.value)
                st = lib.mluOpIndiceConvolutionBackwardDataFromForwardTable(
                    h, d_g, _vp(grad.data_ptr()), d_w, _vp(w.data_ptr()), d_p, _vp(rb.table.data_ptr()),
                    rb.table.numel() * 4, self.num_i64, 0, ly.sub_m, _vp(ws.data_ptr()), self.size.value, d_f,
                    _vp(dx.data_ptr()))
                if st != ops.STATUS_NOT_SUPPORTED:
                    ops.check("mluOpIndiceConvolutionBackwardDataFromForwardTable", st)
                    grad = dx
                    continue
            if reuse_tables and K <= 128:
                if getattr(rb, "input_table", None) is None:
                    size = ctypes.c_size_t(0)
                    ops.check("mluOpGetIndiceInputNeighbourTableSize",
                              lib.mluOpGetIndiceInputNeighbourTableSize(h, d_p, ctypes.byref(size)))
                    rb.input_table = torch.empty((size.value // 4,), dtype=torch.int32, device=self.device)
                    ops.check("mluOpBuildIndiceInputNeighbourTable",
                              lib.mluOpBuildIndiceInputNeighbourTable(h, d_p, _vp(rec.pairs.data_ptr()), self.num_i64,
                                                                      n_out, _vp(rb.input_table.data_ptr()),
                                                                      size.value))
                ops.check("mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize",
                          lib.mluOpGetIndiceConvolutionBackwardDataFromTableWorkspaceSize(
                              h, d_g, d_w, d_p, d_f, self.num_i64, 0, ctypes.byref(self.size)))
                ws = self.workspace.get(self.size.value)
                ops.check("mluOpIndiceConvolutionBackwardDataFromTable",
                          lib.mluOpIndiceConvolutionBackwardDataFromTable(
                              h, d_g, _vp(grad.data_ptr()), d_w, _vp(w.data_ptr()), d_p,
                              _vp(rb.input_table.data_ptr()), rb.input_table.numel() * 4, self.num_i64, 0, ly.sub_m,
                              _vp(ws.data_ptr()), self.size.value, d_f, _vp(dx.data_ptr())))
                grad = dx
                continue
            ops.check("mluOpGetIndiceConvolutionBackwardDataWorkspaceSize",
                      lib.mluOpGetIndiceConvolutionBackwardDataWorkspaceSize(h, d_g, d_w, d_p, d_f, self.num_i64, 0,
                                                                             ctypes.byref(self.size)))
            ws = self.workspace.get(self.size.value)
            ops.check("mluOpIndiceConvolutionBackwardData",
                      lib.mluOpIndiceConvolutionBackwardData(h, d_g, _vp(grad.data_ptr()), d_w, _vp(w.data_ptr()), d_p,
                                                             _vp(rec.pairs.data_ptr()), self.num_i64, 0, ly.sub_m,
                                                             _vp(ws.data_ptr()), self.size.value, d_f,
                                                             _vp(dx.data_ptr())))
            grad = dx
        return grad, filter_grads


def roofline_bytes_and_flops(records, elem_size):
    """Algorithmic bytes and flops of a run, from its actual pair counts.

    Per convolution: P = sum_k indice_num[k]; flops = 2*P*Ci*Co; bytes =
    P*(Ci+Co)*elem + 8*P (gathered input rows, scattered output rows, two int32
    ids per pair).  Per rulebook: 16*L (indices) + 8*K*L (indice_pairs incl. -1
    tails) + 16*N_out (out_indices) + 4*K (indice_num).
    """
    conv = []
    pairs_bytes = 0
    for rec in records:
        ly = rec.layer
        P = int(sum(rec.indice_num))
        conv.append(dict(P=P, flops=2 * P * ly.ci * ly.co, bytes=P * (ly.ci + ly.co) * elem_size + 8 * P,
                         ci=ly.ci, co=ly.co, n_in=rec.n_in, n_out=rec.n_out, sub_m=ly.sub_m))
        if rec.new_rulebook:
            pairs_bytes += 16 * rec.n_in + 8 * ly.kernel_volume * rec.n_in + 16 * rec.n_out + 4 * ly.kernel_volume
    return conv, pairs_bytes
