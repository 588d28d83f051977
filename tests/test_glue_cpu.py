"""Host-side glue around the layer step: collation, staging order, the runner's call sequence."""
import pytest
import torch

from elmo_b200 import glue


def _reference_collate_labels(label_lists):
    # data.py:24-32 restated: list of (row, label) tuples through a float tensor
    pairs = []
    for i, l in enumerate(label_lists):
        pairs += [(i, lbl) for lbl in l]
    return torch.Tensor(pairs).to(torch.int32).contiguous()


def test_collate_labels_matches_the_reference_collate():
    g = torch.Generator().manual_seed(0)
    lists = [torch.randint(0, 670091, (int(n),), generator=g).tolist()
             for n in torch.randint(0, 9, (64,), generator=g)]
    got = glue.collate_labels(lists, pin=False)
    want = _reference_collate_labels(lists)
    assert got.dtype == torch.int32 and got.shape == want.shape
    assert torch.equal(got, want)


def test_collate_labels_empty_and_large_ids():
    assert glue.collate_labels([[], []], pin=False).shape == (0, 2)
    big = 2 ** 24 + 1                       # not representable in float32: the reference would round it
    got = glue.collate_labels([[big], [], [3, big + 2]], pin=False)
    assert got.tolist() == [[0, big], [2, 3], [2, big + 2]]


def test_collate_tuple_layout():
    batch = [(torch.arange(4), torch.ones(4, dtype=torch.long), [5, 7]),
             (torch.arange(4) + 10, torch.zeros(4, dtype=torch.long), [1])]
    tok, mask, lab = glue.collate(batch)
    assert tok.shape == (2, 4) and mask.shape == (2, 4)
    assert lab.tolist() == [[0, 5], [0, 7], [1, 1]]


def test_stager_keeps_order_and_checks_capacity():
    st = glue.StepStager("cpu", label_capacity=8, embed_shape=(4, 3), embed_dtype=torch.float32)
    a = torch.tensor([[0, 1], [1, 2]], dtype=torch.int32)
    b = torch.tensor([[0, 9]], dtype=torch.int32)
    st.put(a, torch.ones(4, 3))
    st.put(b, torch.full((2, 3), 2.0))
    with pytest.raises(RuntimeError):
        st.put(a)
    la, xa = st.get()
    assert torch.equal(la, a) and xa.shape == (4, 3) and float(xa.sum()) == 12.0
    st.release()
    lb, xb = st.get()
    assert torch.equal(lb, b) and xb.shape == (2, 3) and float(xb.sum()) == 12.0
    with pytest.raises(RuntimeError):
        st.get()
    with pytest.raises(ValueError):
        st.put(torch.zeros(9, 2, dtype=torch.int32))
    with pytest.raises(ValueError):
        st.put(torch.zeros(2, 2, dtype=torch.int64))


class _FakeLayer:
    def __init__(self, d):
        self.grad_input = torch.zeros(8, d)
        self.calls = []

    def xfc_forward_backward(self, embed, labels, xmc_lr, skip_loss=True):
        self.calls.append((tuple(embed.shape), int(labels.shape[0]), xmc_lr[0], skip_loss))
        self.grad_input[:embed.shape[0]] = 4.0
        return 0 if skip_loss else 1.5


def test_train_step_scales_the_gradient_and_backpropagates():
    enc = torch.nn.Linear(5, 3, bias=False)
    x = torch.randn(6, 5)
    out = enc(x)
    layer = _FakeLayer(3)
    labels = torch.zeros(2, 2, dtype=torch.int32)
    loss = glue.xmc_train_step(layer, out, labels, [0.05], grad_accum_step=4, skip_loss=False)
    assert loss == 1.5 and layer.calls == [((6, 3), 2, 0.05, False)]
    # d(out)/d(weight): grad_weight = g^T x with g = 4 / 4 = 1 everywhere
    assert torch.allclose(enc.weight.grad, torch.ones(6, 3).t() @ x)
