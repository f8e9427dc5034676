"""Host-facing inference loop: pinned host images in, host logits out, with the next
batch's host-to-device copy and the previous batch's logits gather + device-to-host copy
overlapped with the current batch's compute.

The reference's eval loop copies each batch and then runs the model on the same stream
(``vtpack/engine/engine.py:113-118``); here the input copy runs on its own stream into a
second device buffer, and the logits leave on a third stream (NCCL all-gather when there is
more than one rank, then the copy to pinned host memory), so the copy engines, NVLink and
the SMs work at the same time.  Every buffer is double-buffered; a slot is reused only after
the stream that read it last has passed an event.
"""
import torch


class LogitsGather:
    """All-gather of each step's ``[B, classes]`` logits on a side stream.

    ``start(slot)`` is called on the compute stream right after the forward that wrote
    ``local[slot]``; the collective (and, when ``host`` buffers are given, the device-to-host
    copy) then runs on the side stream while the compute stream goes on with the next batch.
    ``local[slot]`` may be written again once ``reusable(slot)`` has been called on the stream
    that will write it."""

    def __init__(self, batch, num_classes, device, world=1, group=None, to_host=False):
        self.device = torch.device(device)
        self.world, self.group = world, group
        self.stream = torch.cuda.Stream(self.device)
        self.local = [torch.empty(batch, num_classes, device=self.device) for _ in range(2)]
        self.gathered = ([torch.empty(batch * world, num_classes, device=self.device) for _ in range(2)]
                         if world > 1 else None)
        self.host = ([torch.empty(batch * world, num_classes).pin_memory() for _ in range(2)] if to_host else None)
        self.ready = [torch.cuda.Event() for _ in range(2)]     # forward of the slot finished (compute stream)
        self.done = [torch.cuda.Event() for _ in range(2)]      # gather (+ host copy) of the slot finished
        for ev in self.done:
            ev.record(torch.cuda.current_stream(self.device))

    def reusable(self, slot, stream=None):
        """Makes `stream` (default: current) wait until the slot's previous gather has read local[slot]."""
        (stream or torch.cuda.current_stream(self.device)).wait_event(self.done[slot])

    def start(self, slot):
        import torch.distributed as dist
        cur = torch.cuda.current_stream(self.device)
        self.ready[slot].record(cur)
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(self.ready[slot])
            src = self.local[slot]
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered[slot], src, group=self.group)
                src = self.gathered[slot]
            if self.host is not None:
                self.host[slot].copy_(src, non_blocking=True)
            self.done[slot].record(self.stream)
        return src

    def wait_all(self):
        """Makes the current stream wait for both slots' outstanding gathers."""
        cur = torch.cuda.current_stream(self.device)
        for ev in self.done:
            cur.wait_event(ev)


class HostPipeline:
    def __init__(self, model, batch: int, img_size: int, device, num_classes: int = 1000, group=None,
                 world: int = 1, image_dtype=torch.float32, use_graph: bool = False):
        self.model = model
        self.use_graph = use_graph
        self.device = torch.device(device)
        self.copy_stream = torch.cuda.Stream(self.device)
        self.dev_in = [torch.empty(batch, 3, img_size, img_size, device=self.device, dtype=image_dtype)
                       for _ in range(2)]
        self.out = LogitsGather(batch, num_classes, self.device, world=world, group=group, to_host=True)
        self.dev_logits, self.host_logits = self.out.local, self.out.host
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        self.group, self.world = group, world
        self.h2d_bytes = self.dev_in[0].numel() * self.dev_in[0].element_size()
        self.d2h_bytes = self.host_logits[0].numel() * 4

    def _stage(self, host_images, slot):
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])     # the previous user of this buffer is done
            self.dev_in[slot].copy_(host_images, non_blocking=True)
            self.copied[slot].record(self.copy_stream)

    def run(self, host_batches):
        """host_batches: sequence of pinned [B,3,S,S] tensors of the pipeline's image dtype.  Returns the host
        logits of the last batch (each batch's logits land in a pinned buffer)."""
        main = torch.cuda.current_stream(self.device)
        n = len(host_batches)
        if n == 0:
            return None
        for s in range(2):
            self.consumed[s].record(main)
        self._stage(host_batches[0], 0)
        last = None
        for i in range(n):
            slot = i & 1
            if i + 1 < n:
                self._stage(host_batches[i + 1], slot ^ 1)
            main.wait_event(self.copied[slot])
            self.out.reusable(slot, main)            # the gather of two batches ago has read this logits buffer
            if self.use_graph:
                self.model.forward_graph(self.dev_in[slot], self.dev_logits[slot])
            else:
                self.model(self.dev_in[slot], logits_out=self.dev_logits[slot])
            self.consumed[slot].record(main)
            self.out.start(slot)
            last = self.host_logits[slot]
        self.out.wait_all()
        main.synchronize()
        return last
