"""Streaming inference: host image batches in, per-image detections out, with the copies overlapped.

The counterpart of the loop in the reference's inference script (KAD-CNet/inference/infer_dior.py:39-60: load a batch,
`/255`, model, non_max_suppression, collect), arranged for throughput on one GPU: the host-to-device copy of batch i+1
runs on a copy stream while batch i is in the forward graph, the batched NMS of batch i runs on a third stream while batch i+1
is in the forward graph, the detections come back as one padded tensor plus counts (one device-to-host copy per batch, no
per-image synchronisation), and the host only waits for batch i-1 while batch i is running. There is no CPU path: the model must be a B200 engine (`load_model(..., backend='optimized')`).
"""
import torch

from kadconv import ops

from .runtime import StaticGraph


class DetectionPipeline:
    """pipeline = DetectionPipeline(fast_model, (mb, 3, H, W)); for dets in pipeline.run(batches): ...

    `batches`: an iterable of uint8 tensors [mb,3,H,W] in pinned host memory (or already on the device).
    Yields, per batch and in order, a list of mb float32 tensors [n_i, 6] (x1, y1, x2, y2, confidence, class) on the host;
    with to_host=False the padded device tensors (dets [mb,max_det,6], counts [mb]) of a double buffer instead: consume them
    before the batch after the next one is submitted.

    Streams: the copy stream uploads batch i+1 while batch i is in the forward graph on the main stream, and the
    post-processing stream runs the batched NMS (one CTA per image: it leaves most of the GPU idle) and the device-to-host copy
    of batch i while batch i+1 is already in the forward graph. The prediction tensor is copied out of the graph's output buffer
    (40 MB per 64 images, a few microseconds) so that the next replay cannot overwrite what NMS still reads.
    """

    def __init__(self, fast_model, batch_shape, conf_thres=0.25, iou_thres=0.45, max_det=300, device=None, splits=1):
        """splits > 1: the forward of a batch runs as `splits` CUDA graphs over equal parts of it, replayed side by side on
        their own streams (the layers on the small feature maps of the detector do not fill the GPU; two half-batches
        interleave better than one batch). The results are the same bit for bit."""
        self.device = torch.device(device) if device is not None else fast_model.device
        if self.device.type != 'cuda':
            raise RuntimeError('DetectionPipeline needs a CUDA device (there is no CPU path)')
        self.conf, self.iou, self.max_det = conf_thres, iou_thres, max_det
        self.shape = tuple(batch_shape)
        mb = self.shape[0]
        if splits < 1 or mb % splits:
            raise ValueError(f'splits = {splits} does not divide the batch of {mb}')
        self.splits, self.part = splits, mb // splits
        with torch.cuda.device(self.device):
            self.stage = [torch.empty(self.shape, dtype=torch.uint8, device=self.device) for _ in range(2)]
            self.graphs = [StaticGraph(lambda u8: fast_model(u8)[0], self.stage[0][k * self.part:(k + 1) * self.part]) for k in range(splits)]
            self.graph = self.graphs[0]
            self.fwd_streams = [torch.cuda.Stream(self.device) for _ in range(splits)] if splits > 1 else []
            self.copy_stream = torch.cuda.Stream(self.device)
            self.post_stream = torch.cuda.Stream(self.device)
            out = self.graph.output
            self.pred = [torch.empty((mb,) + tuple(out.shape[1:]), dtype=out.dtype, device=self.device) for _ in range(2)]
            self.dets = [torch.zeros((mb, max_det, 6), dtype=torch.float32, device=self.device) for _ in range(2)]
            self.counts = [torch.zeros((mb,), dtype=torch.int32, device=self.device) for _ in range(2)]
            self.status_host = [torch.zeros(4, dtype=torch.int32).pin_memory() for _ in range(2)]
            self.out_dets = [torch.empty((mb, max_det, 6), dtype=torch.float32).pin_memory() for _ in range(2)]
            self.out_counts = [torch.empty((mb,), dtype=torch.int32).pin_memory() for _ in range(2)]
            self.h2d_done = [torch.cuda.Event() for _ in range(2)]
            self.stage_free = [torch.cuda.Event() for _ in range(2)]
            self.fwd_done = [torch.cuda.Event() for _ in range(2)]
            self.result_ready = [torch.cuda.Event() for _ in range(2)]

    def _upload(self, batch, slot):
        if tuple(batch.shape) != self.shape or batch.dtype != torch.uint8:
            raise ValueError(f'expected a uint8 batch of shape {self.shape}, got {tuple(batch.shape)} {batch.dtype}')
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.stage_free[slot])        # the previous user of this staging buffer has consumed it
            self.stage[slot].copy_(batch, non_blocking=True)
            self.h2d_done[slot].record(self.copy_stream)

    def _collect(self, slot, to_host):
        if not to_host:
            return self.dets[slot], self.counts[slot]
        self.result_ready[slot].synchronize()
        ops.raise_if_aborted(self.status_host[slot].tolist(), ops.status_word(self.device).zero_)
        dets, counts = self.out_dets[slot], self.out_counts[slot].tolist()
        return [dets[i, :n].clone() for i, n in enumerate(counts)]

    @torch.no_grad()
    def run(self, batches, to_host=True):
        main = torch.cuda.current_stream(self.device)
        post = self.post_stream
        for ev in self.stage_free:
            ev.record(main)
        for ev in self.result_ready:
            ev.record(main)
        it = iter(batches)
        nxt = next(it, None)
        if nxt is None:
            return
        self._upload(nxt, 0)
        i, pending = 0, None
        while nxt is not None:
            slot = i & 1
            following = next(it, None)
            if following is not None:
                self._upload(following, slot ^ 1)                      # overlaps the forward below
            main.wait_event(self.h2d_done[slot])
            if self.splits == 1:
                self.graph.input.copy_(self.stage[slot], non_blocking=True)
                self.stage_free[slot].record(main)
                self.graph.graph.replay()
                main.wait_event(self.result_ready[slot])               # post-processing of batch i-2 no longer reads this slot
                self.pred[slot].copy_(self.graph.output, non_blocking=True)
            else:
                main.wait_event(self.result_ready[slot])
                for k, (g, st) in enumerate(zip(self.graphs, self.fwd_streams)):
                    part = slice(k * self.part, (k + 1) * self.part)
                    st.wait_stream(main)
                    with torch.cuda.stream(st):
                        g.input.copy_(self.stage[slot][part], non_blocking=True)
                        g.graph.replay()
                        self.pred[slot][part].copy_(g.output, non_blocking=True)
                for st in self.fwd_streams:
                    main.wait_stream(st)
                self.stage_free[slot].record(main)
            self.fwd_done[slot].record(main)
            with torch.cuda.stream(post):                              # overlaps the forward of the next batch
                post.wait_event(self.fwd_done[slot])
                ops.nms_batched(self.pred[slot], self.conf, self.iou, self.max_det, out=(self.dets[slot], self.counts[slot]))
                if to_host:
                    self.out_dets[slot].copy_(self.dets[slot], non_blocking=True)
                    self.out_counts[slot].copy_(self.counts[slot], non_blocking=True)
                    self.status_host[slot].copy_(ops.status_word(self.device), non_blocking=True)
                self.result_ready[slot].record(post)
            if pending is not None:                                    # results of the batch before this one (its slot is `slot ^ 1`)
                yield self._collect(pending, to_host)
            pending = slot
            nxt = following
            i += 1
        yield self._collect(pending, to_host)
        main.wait_event(self.result_ready[0]); main.wait_event(self.result_ready[1])
        if to_host:
            ops.check_status(self.device)
