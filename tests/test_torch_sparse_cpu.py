"""Host-side behaviour of the PyTorch modules that needs no GPU: parameter shapes,
geometry rules, and the refusal to run on CPU tensors."""
import importlib

import pytest
import torch


@pytest.fixture(scope="module")
def sp(pkg):
    return importlib.import_module("mluops_b200.torch_sparse")


def test_parameter_shapes_and_geometry(sp):
    l = sp.SparseConv3d(4, 16, (3, 1, 1), stride=(2, 1, 1), padding=0, bias=True)
    assert tuple(l.weight.shape) == (3, 1, 1, 4, 16) and tuple(l.bias.shape) == (16,)
    s = sp.SubMConv3d(16, 32, 3, indice_key="k")
    assert s.padding == [1, 1, 1] and s.subm and s.indice_key == "k"
    with pytest.raises(AssertionError):
        sp.SubMConv3d(16, 32, 2)
    with pytest.raises(AssertionError):
        sp.SparseConvolution(16, 32, 3, stride=2, subm=True)


def test_cpu_tensors_are_refused(sp):
    with pytest.raises(AssertionError):
        sp.SparseConvTensor(torch.zeros(3, 4), torch.zeros((3, 4), dtype=torch.int32), [2, 2, 2], 1)
