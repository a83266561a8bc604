"""CPU: the import surface the reference's scripts expect from `bqq_modules`, its model builder
running unchanged on this package's classes, reference-made pickles, and the training-time
helpers (PartialBQQLinear, merge_*).  No GPU work: forwards of BinaryQuadratic are not called here
(they need the device); dense weights come from get_weight's torch route."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn as nn

import bqq_b200
from oracle import bqq_oracle as O
from tests.helpers import GOLDEN, synth_layer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_root():
    """Checkout of the reference project: $BQQ_REFERENCE_ROOT, or a `reference` directory beside
    the repository.  None when absent (the tests that need it are skipped)."""
    for cand in (os.environ.get('BQQ_REFERENCE_ROOT'), os.path.join(os.path.dirname(ROOT), 'reference')):
        if cand and os.path.isdir(os.path.join(cand, 'neural_network_compression', 'lm')):
            return cand
    return None


def _patches_from_golden(io, name):
    out, n = [], 0
    while f'{name}/{n}/idx' in io:
        i, j, k = (int(v) for v in io[f'{name}/{n}/idx'])
        out.append(dict(patch_row=i, patch_col=j, bit_idx=k, coeff=torch.from_numpy(io[f'{name}/{n}/coeff']),
                        mat1=torch.from_numpy(io[f'{name}/{n}/mat1']).float(),
                        mat2=torch.from_numpy(io[f'{name}/{n}/mat2']).float()))
        n += 1
    return out


def _golden_io():
    g = np.load(os.path.join(GOLDEN, 'ref_model_io.npz'))
    return {k: g[k] for k in g.files}


def test_reference_import_list_resolves():
    """The exact names lm/build_bqq_model.py:57-65, lm/benchmark_inference.py:21 and the packed-layer
    scripts import."""
    bqq_b200.install()
    from bqq_modules import (BinaryQuadratic, PackedBinaryQuadratic, PartialBQQLinear, get_matrices,  # noqa: F401
                             merge_binary_quadratic, merge_binaryquadratic_recursive, pack_binaryquadratic_model)
    import bqq_cuda_ext
    assert callable(bqq_cuda_ext._get_ext().bqq_forward) and callable(bqq_cuda_ext.bqq_forward)
    assert BinaryQuadratic is bqq_b200.BinaryQuadratic


def test_vision_layers_fail_with_a_clear_message(monkeypatch):
    bqq_b200.install()
    monkeypatch.delenv('BQQ_REFERENCE_SRC', raising=False)
    monkeypatch.setattr(bqq_b200.bqq_modules, '_reference_module', None)
    with pytest.raises(ImportError, match='BQQ_REFERENCE_SRC'):
        from bqq_modules import BQQLinear  # noqa: F401


def test_reference_pickles_load_onto_this_package():
    bqq_b200.install()
    io = _golden_io()
    for fname, cls in (('ref_model_bq.pth', bqq_b200.BinaryQuadratic),
                       ('ref_model_bq-packed.pth', bqq_b200.PackedBinaryQuadratic)):
        model = torch.load(os.path.join(GOLDEN, fname), weights_only=False)
        assert type(model.fc1) is cls and type(model.fc2) is cls and isinstance(model.head, nn.Linear)
        assert (model.fc1.bit_width, model.fc1.row_width, model.fc1.col_width) == (2, 3, 2)
        assert (model.fc1.y_row, model.fc1.inter_dimension, model.fc1.z_col) == (32, 16, 32)
        keys = list(model.fc1.state_dict().keys())
        if cls is bqq_b200.BinaryQuadratic:
            assert keys == ['a', 'b', 'c', 'd', 'bias', 'Y', 'Z']
            W = model.fc1.get_weight(torch.float32)          # torch route, module is on the host
            assert np.abs(W.detach().numpy() - io['fc1_weight']).max() < 1e-6
        else:
            assert keys == ['a', 'b', 'c', 'd', 'bias', 'Y_packed', 'Z_packed', 'Y_sum_i16', 'Z_sum_i16']


def _write_patch_dir(tmp_path, io, consolidated):
    root = tmp_path / ('merged' if consolidated else 'per_patch')
    (root / '_consolidated').mkdir(parents=True) if consolidated else root.mkdir()
    for name in ('fc1.weight', 'fc2.weight'):
        patches = _patches_from_golden(io, name)
        if consolidated:
            torch.save(patches, root / '_consolidated' / f'{name}.pth')
        else:   # the quantiser's per-patch files: <name>_row<i>_col<j>.pth, each a list of dicts
            cells = {}
            for p in patches:
                cells.setdefault((p['patch_row'], p['patch_col']), []).append(p)
            for (i, j), lst in cells.items():
                torch.save(lst, root / f'{name}_row{i}_col{j}.pth')
    return root


def _small_model():
    from collections import OrderedDict
    return nn.Sequential(OrderedDict(fc1=nn.Linear(64, 96, bias=True), act=nn.Tanh(),
                                     fc2=nn.Linear(96, 64, bias=False), head=nn.Linear(64, 8, bias=False)))


@pytest.mark.parametrize('consolidated', [True, False])
def test_own_replace_reads_the_reference_patch_layouts(tmp_path, consolidated):
    io = _golden_io()
    root = _write_patch_dir(tmp_path, io, consolidated)
    model = bqq_b200.replace_linear_with_bqq(_small_model(), str(root), 2)
    assert isinstance(model.fc1, bqq_b200.BinaryQuadratic) and isinstance(model.head, nn.Linear)
    assert model.fc1.bit_width == 2                       # the third bit layer of fc1's patches is dropped
    W = model.fc1.get_weight(torch.float32).detach().numpy()
    assert np.abs(W - io['fc1_weight']).max() < 1e-6
    planes = bqq_b200.replace_linear_with_bqq(_small_model(), str(root), 2, planes_only=True)
    assert isinstance(planes.fc2, bqq_b200.PlaneBinaryQuadratic)


def test_reference_builder_runs_unchanged_on_this_package(tmp_path, monkeypatch):
    """lm/build_bqq_model.py imported as it is, with this package standing in for bqq_modules:
    replace_linear_with_bqq, save (torch.save of the model), pack_existing_model and
    dequantize_bqq_model."""
    ref = _reference_root()
    if ref is None:
        pytest.skip('no checkout of the reference project (set BQQ_REFERENCE_ROOT)')
    bqq_b200.install()
    lm = os.path.join(ref, 'neural_network_compression', 'lm')
    monkeypatch.syspath_prepend(lm)
    sys.modules.pop('build_bqq_model', None)
    B = importlib.import_module('build_bqq_model')
    try:
        assert B.BinaryQuadratic is bqq_b200.BinaryQuadratic
        assert B.PartialBQQLinear is bqq_b200.PartialBQQLinear
        io = _golden_io()
        root = _write_patch_dir(tmp_path, io, True)
        model = B.replace_linear_with_bqq(_small_model(), str(root), 2, show_tqdm=False)
        assert type(model.fc1) is bqq_b200.BinaryQuadratic and type(model.fc2) is bqq_b200.BinaryQuadratic
        assert isinstance(model.head, nn.Linear)
        assert np.abs(model.fc1.get_weight(torch.float32).detach().numpy() - io['fc1_weight']).max() < 1e-6
        path = tmp_path / 'model.pth'
        torch.save(model, path)                               # what save_bqq_model does (:189-190)
        packed_path = B.pack_existing_model(path)
        packed = torch.load(packed_path, weights_only=False)
        assert type(packed.fc1) is bqq_b200.PackedBinaryQuadratic
        ref_packed = torch.load(os.path.join(GOLDEN, 'ref_model_bq-packed.pth'), weights_only=False)
        for key, val in ref_packed.state_dict().items():      # same bytes as the reference's own packing
            if key.endswith('bias') or key.startswith('head'):    # the Linear's own random initialisation
                continue
            assert torch.equal(val, packed.state_dict()[key]), key
        dense = B.dequantize_bqq_model(torch.load(path, weights_only=False), dtype=torch.float32)
        assert isinstance(dense.fc1, nn.Linear)
        assert np.abs(dense.fc1.weight.detach().numpy() - io['fc1_weight']).max() < 1e-6
    finally:
        sys.modules.pop('build_bqq_model', None)
        sys.modules.pop('compressed_data', None)


def test_partial_layer_matches_reference_semantics():
    torch.manual_seed(0)
    lin = nn.Linear(64, 96, bias=True)
    part = bqq_b200.PartialBQQLinear(lin.weight.data, lin.bias.data, group_size=32, bit_width=2)
    X = torch.randn(5, 64)
    assert torch.allclose(part(X), lin(X), atol=1e-6)        # nothing quantised yet: the float layer
    Y, Z, A, _, _ = synth_layer(2, 3, 2, 32, 32, 16, 1, seed=4)
    part.quantize_patch(1, 0, A[:, 1, 0], Y[:, 1, 0].float(), Z[:, 1, 0].float())
    a, b, c, d = O.split_coefficients(A.numpy())
    Wq = O.dense_weight(Y.numpy(), Z.numpy(), a, b, c, d)
    W_mixed = lin.weight.data.clone().numpy()
    W_mixed[32:64, 0:32] = Wq[32:64, 0:32]
    expect = X.numpy() @ W_mixed.T + lin.bias.data.numpy()
    assert np.abs(part(X).detach().numpy() - expect).max() < 1e-4
    # gradients: the quantised patch feeds a..d, the rest feeds float_weight
    part(X).sum().backward()
    assert part.a.grad[:, 1, 0].abs().sum() > 0 and part.a.grad[:, 0, 0].abs().sum() == 0
    assert part.float_weight.grad[32:64, 0:32].abs().sum() == 0 and part.float_weight.grad[0:32].abs().sum() > 0
    with pytest.raises(RuntimeError, match='still unquantized'):
        part.to_binaryquadratic()
    for i in range(3):
        for j in range(2):
            part.quantize_patch(i, j, A[:, i, j], Y[:, i, j].float(), Z[:, i, j].float())
    bq = part.to_binaryquadratic()
    direct = bqq_b200.BinaryQuadratic(Y.float(), Z.float(), A, bias=lin.bias.data)
    assert type(bq) is bqq_b200.BinaryQuadratic
    for (k1, v1), (k2, v2) in zip(bq.state_dict().items(), direct.state_dict().items()):
        assert k1 == k2 and torch.equal(v1, v2), k1


def test_partial_layer_against_the_reference_class():
    ref = _reference_root()
    if ref is None:
        pytest.skip('no checkout of the reference project (set BQQ_REFERENCE_ROOT)')
    spec = importlib.util.spec_from_file_location(
        '_ref_bqq_modules', os.path.join(ref, 'neural_network_compression', 'src', 'bqq_modules.py'))
    rm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rm)
    torch.manual_seed(1)
    lin = nn.Linear(64, 64, bias=True)
    mine = bqq_b200.PartialBQQLinear(lin.weight.data, lin.bias.data, 32, 2)
    theirs = rm.PartialBQQLinear(lin.weight.data, lin.bias.data, 32, 2)
    Y, Z, A, _, X = synth_layer(2, 2, 2, 32, 32, 16, 4, seed=6)
    for step, (i, j) in enumerate([(0, 1), (1, 1), (0, 0), (1, 0)]):
        for m in (mine, theirs):
            m.quantize_patch(i, j, A[:, i, j], Y[:, i, j].float(), Z[:, i, j].float())
        assert torch.allclose(mine(X), theirs(X), atol=1e-6), step
    assert list(mine.state_dict().keys()) == list(theirs.state_dict().keys())
    for k, v in theirs.to_binaryquadratic().state_dict().items():
        assert torch.equal(v, mine.to_binaryquadratic().state_dict()[k]), k


def test_merge_appends_bit_layers():
    Yq, Zq, Aq, bias, _ = synth_layer(2, 2, 3, 32, 32, 16, 1, seed=7, bias=True)
    Yd, Zd, Ad, _, _ = synth_layer(1, 2, 3, 32, 32, 16, 1, seed=8, coef_scale=0.005)
    quant = bqq_b200.BinaryQuadratic(Yq.float(), Zq.float(), Aq, bias=bias)
    diff = bqq_b200.BinaryQuadratic(Yd.float(), Zd.float(), Ad)
    merged = bqq_b200.merge_binary_quadratic(diff, quant)
    assert merged.bit_width == 3 and merged.Y.shape[0] == 3 and torch.equal(merged.bias.data, bias)
    W = merged.get_weight(torch.float32)
    assert torch.allclose(W, quant.get_weight(torch.float32) + diff.get_weight(torch.float32), atol=1e-6)
    mq, md = nn.Sequential(quant, nn.Tanh()), nn.Sequential(diff, nn.Tanh())
    out = bqq_b200.merge_binaryquadratic_recursive(mq, md)
    assert out[0].bit_width == 3
    with pytest.raises(ValueError):
        bqq_b200.merge_binary_quadratic(bqq_b200.BinaryQuadratic(Yd[:, :1].float(), Zd[:, :1].float(), Ad[:, :1]), quant)
