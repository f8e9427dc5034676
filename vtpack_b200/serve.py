"""Host-facing inference loop: pinned host images in, host logits out, with the next
batch's host-to-device copy overlapped with the current batch's compute.

The reference's eval loop copies each batch and then runs the model on the same stream
(``vtpack/engine/engine.py:113-118``); here the copy runs on its own stream into a
second device buffer so the copy engine and the SMs work at the same time.
"""
import torch


class HostPipeline:
    def __init__(self, model, batch: int, img_size: int, device, num_classes: int = 1000, group=None,
                 world: int = 1, image_dtype=torch.float32, use_graph: bool = False):
        self.model = model
        self.use_graph = use_graph
        self.device = torch.device(device)
        self.copy_stream = torch.cuda.Stream(self.device)
        self.dev_in = [torch.empty(batch, 3, img_size, img_size, device=self.device, dtype=image_dtype)
                       for _ in range(2)]
        self.dev_logits = [torch.empty(batch, num_classes, device=self.device) for _ in range(2)]
        self.host_logits = [torch.empty(batch * world, num_classes).pin_memory() for _ in range(2)]
        self.gathered = ([torch.empty(batch * world, num_classes, device=self.device) for _ in range(2)]
                         if world > 1 else None)
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
        import torch.distributed as dist
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
            if self.use_graph:
                self.model.forward_graph(self.dev_in[slot], self.dev_logits[slot])
            else:
                self.model(self.dev_in[slot], logits_out=self.dev_logits[slot])
            self.consumed[slot].record(main)
            src = self.dev_logits[slot]
            if self.world > 1:
                dist.all_gather_into_tensor(self.gathered[slot], src, group=self.group)
                src = self.gathered[slot]
            self.host_logits[slot].copy_(src, non_blocking=True)
            last = self.host_logits[slot]
        main.synchronize()
        return last
