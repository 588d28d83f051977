"""Staging and the runner's call sequence with the real layer on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_staged_steps_equal_direct_steps():
    from elmo_b200 import glue
    from elmo_b200.handle import XmcHandle
    dev = torch.device("cuda", 0)
    L, d, B = 2048, 128, 64
    g = torch.Generator().manual_seed(3)
    w0 = (torch.randn(L, d, generator=g) * 0.25).to(torch.float8_e4m3fn)
    steps = []
    for _ in range(4):
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
        lists = [torch.randint(0, L, (int(n),), generator=g).tolist() for n in torch.randint(1, 6, (B,), generator=g)]
        steps.append((x, glue.collate_labels(lists)))

    def run(staged):
        w = w0.clone().to(dev)
        h = XmcHandle(dev, d, B, "fp8")
        h.bind([w])
        gx = torch.zeros(B, d, dtype=torch.float32, device=dev)
        st = glue.StepStager(dev, label_capacity=B * 8, embed_shape=(B, d)) if staged else None
        if staged:
            st.put(steps[0][1], steps[0][0])
        for i, (x, lab) in enumerate(steps):
            if staged:
                if i + 1 < len(steps):
                    st.put(steps[i + 1][1], steps[i + 1][0])      # next step's copy overlaps this step
                dl, dx = st.get()
            else:
                dl, dx = lab.to(dev), x.to(dev)
            h.step(dx, dl, 0.3, seed=9, step=i, stochastic=True, grad_f32=gx)
            if staged:
                st.release()
        h.check()
        out = w.cpu().view(torch.uint8), gx.cpu()
        h.close()
        return out

    wa, ga = run(False)
    wb, gb = run(True)
    assert torch.equal(wa, wb) and torch.equal(ga, gb)


def test_many_staged_steps_without_host_sync():
    """Forty steps queued back to back (the host runs far ahead of the GPU): every step must see its own
    labels and embeddings, i.e. a pinned slot is not rewritten before the copy that reads it has run."""
    from elmo_b200 import glue
    from elmo_b200.handle import XmcHandle
    dev = torch.device("cuda", 0)
    L, d, B, n_steps = 32768, 256, 256, 40             # a step long enough for the host to get ahead
    g = torch.Generator().manual_seed(8)
    w0 = (torch.randn(L, d, generator=g) * 0.25).to(torch.float8_e4m3fn)
    steps = []
    for _ in range(n_steps):
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
        lab = torch.stack([torch.randint(0, B, (600,), generator=g), torch.randint(0, L, (600,), generator=g)], 1)
        steps.append((x, lab.to(torch.int32)))

    def run(staged):
        w = w0.clone().to(dev)
        h = XmcHandle(dev, d, B, "fp8")
        h.bind([w])
        gx = torch.zeros(n_steps, B, d, dtype=torch.float32, device=dev)
        st = glue.StepStager(dev, label_capacity=1024, embed_shape=(B, d)) if staged else None
        if staged:
            st.put(steps[0][1], steps[0][0])
        for i, (x, lab) in enumerate(steps):
            if staged:
                if i + 1 < n_steps:
                    st.put(steps[i + 1][1], steps[i + 1][0])
                dl, dx = st.get()
            else:
                dl, dx = lab.to(dev), x.to(dev)
            h.step(dx, dl, 0.3, seed=9, step=i, stochastic=True, grad_f32=gx[i])
            if staged:
                st.release()
        h.check()
        out = w.cpu().view(torch.uint8), gx.cpu()
        h.close()
        return out

    wa, ga = run(False)
    wb, gb = run(True)
    assert torch.equal(ga, gb)
    assert torch.equal(wa, wb)
