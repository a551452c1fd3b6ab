"""Operators on HOST buffers: staged copies around the device entry points.

The reference's CPU backend takes host pointers; its nv-gpu backend (and this
library) takes device pointers, so a caller that holds its tensors in host
memory has to move them.  `StagedPipeline` does that the way the PCIe link
wants it: three CUDA streams, one for host-to-device copies, one for the
operator launches, one for device-to-host copies, chained by events per stage.
Uploads of stage i+1 then run under the kernel of stage i and under the
download of its results; the link carries traffic in both directions at once
and a step costs max(upload, download) instead of their sum.

Host tensors should be pinned (`tensor.pin_memory()`), otherwise the copies
are staged by the driver and do not overlap.

Buffer hazards across repeated `run()` calls are covered by events too:
  * an upload into a device buffer waits until the last kernel that read the
    buffer, and the last download from it (in-place operators), are done;
  * a kernel waits until the previous download of its output buffers is done.
"""


class Stage:
    """One operator call.  `uploads` / `downloads` are lists of (device_tensor,
    host_tensor); `launch(stream_ptr)` enqueues the operator on that stream."""

    def __init__(self, name, uploads, launch, downloads):
        self.name, self.uploads, self.launch, self.downloads = name, list(uploads), launch, list(downloads)


class StagedPipeline:
    def __init__(self, stages, device):
        import torch

        self.torch, self.device, self.stages = torch, device, list(stages)
        self.s_in = torch.cuda.Stream(device=device)
        self.s_run = torch.cuda.Stream(device=device)
        self.s_out = torch.cuda.Stream(device=device)
        n = len(self.stages)
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_run = [torch.cuda.Event() for _ in range(n)]
        self.ev_out = [torch.cuda.Event() for _ in range(n)]
        self.ran = False
        self.h2d_bytes = sum(h.numel() * h.element_size() for st in self.stages for _, h in st.uploads)
        self.d2h_bytes = sum(h.numel() * h.element_size() for st in self.stages for _, h in st.downloads)

    def run(self):
        """Enqueue one pass over all stages; returns without waiting."""
        torch = self.torch
        for i, st in enumerate(self.stages):
            with torch.cuda.stream(self.s_in):
                if self.ran:  # the buffers' previous readers
                    self.s_in.wait_event(self.ev_run[i])
                    if st.downloads:
                        self.s_in.wait_event(self.ev_out[i])
                for dev_t, host_t in st.uploads:
                    dev_t.copy_(host_t, non_blocking=True)
                self.ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                if self.ran and st.downloads:
                    self.s_run.wait_event(self.ev_out[i])
                st.launch(self.s_run.cuda_stream)
                self.ev_run[i].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[i])
                for dev_t, host_t in st.downloads:
                    host_t.copy_(dev_t, non_blocking=True)
                self.ev_out[i].record(self.s_out)
        self.ran = True

    def join(self, stream):
        """Make `stream` wait for everything enqueued so far."""
        for s in (self.s_in, self.s_run, self.s_out):
            ev = self.torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)

    def fork(self, stream):
        """Make the pipeline's streams wait for what `stream` holds now."""
        ev = self.torch.cuda.Event()
        ev.record(stream)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(ev)

    def synchronize(self):
        for s in (self.s_in, self.s_run, self.s_out):
            s.synchronize()
