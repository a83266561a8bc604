"""Generate whole-module pickles with the UNMODIFIED reference, as its model builder writes them.

    python tests/golden/make_pickles.py /path/to/reference

Steps, all through the reference's own code (lm/build_bqq_model.py, lm/compressed_data.py,
src/bqq_modules.py):
  1. patch dicts {patch_row, patch_col, coeff, mat1, mat2, bit_idx} for the two Linear layers of a
     small torch model are written in the quantiser's consolidated layout
     `<dir>/_consolidated/<name>.weight.pth` (quantizer.py:883-895, lm/compressed_data.py:152-191);
  2. replace_linear_with_bqq(model, weights_dir, bit_width) (lm/build_bqq_model.py:79-112) swaps the
     Linears for the reference's BinaryQuadratic; torch.save(model) as save_bqq_model does (:189-190)
     -> ref_model_bq.pth;
  3. pack_existing_model (:259-279) -> ref_model_bq-packed.pth (PackedBinaryQuadratic layers);
  4. inputs and the reference's fp32 outputs of the unpacked model -> ref_model_io.npz, together with
     the patch dicts themselves (so that tests can rebuild the patch directory without the reference).

The tests read only the files written here, never the reference checkout.
"""
import os
import sys
import tempfile
from collections import OrderedDict

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def make_patches(gen, out_f, in_f, P, Q, r, bits):
    patches = []
    for i in range(out_f // P):
        for j in range(in_f // Q):
            for k in range(bits):
                patches.append(dict(patch_row=i, patch_col=j, bit_idx=k,
                                    coeff=torch.randn(4, generator=gen) * (0.02 if k < 2 else 0.005),
                                    mat1=(torch.rand(P, r, generator=gen) > 0.5).float(),
                                    mat2=(torch.rand(r, Q, generator=gen) > 0.5).float()))
    return patches


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = os.path.join(sys.argv[1], 'neural_network_compression')
    sys.path.insert(0, os.path.join(ref, 'src'))
    sys.path.insert(0, os.path.join(ref, 'lm'))
    import build_bqq_model as B                      # the reference's builder, unmodified
    import bqq_modules as bm
    bm.PackedBinaryQuadratic.use_packed_kernel = False

    gen = torch.Generator().manual_seed(11)
    model = nn.Sequential(OrderedDict(
        fc1=nn.Linear(64, 96, bias=True), act=nn.Tanh(), fc2=nn.Linear(96, 64, bias=False),
        head=nn.Linear(64, 8, bias=False)))          # 'head' must be skipped by the replacement
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.1)
    layers = {'fc1.weight': make_patches(gen, 96, 64, 32, 32, 16, 3),     # a third bit layer that bit_width=2 drops
              'fc2.weight': make_patches(gen, 64, 96, 32, 32, 16, 2)}
    X = torch.randn(3, 64, generator=gen)

    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, '_consolidated'))
        for name, patches in layers.items():
            torch.save(patches, os.path.join(tmp, '_consolidated', name + '.pth'))
        model = B.replace_linear_with_bqq(model, tmp, 2, show_tqdm=False)
    assert type(model.fc1).__module__ == 'bqq_modules' and isinstance(model.head, nn.Linear)
    with torch.no_grad():
        y = model(X)
        W1 = model.fc1.get_weight(torch.float32)
    out = os.path.join(HERE, 'ref_model_bq.pth')
    torch.save(model, out)
    B.pack_existing_model(out)                       # writes ref_model_bq-packed.pth beside it
    flat = {}
    for name, patches in layers.items():
        for n, p in enumerate(patches):
            for key in ('coeff', 'mat1', 'mat2'):
                flat[f'{name}/{n}/{key}'] = p[key].numpy().astype(np.float32 if key == 'coeff' else np.uint8)
            flat[f'{name}/{n}/idx'] = np.array([p['patch_row'], p['patch_col'], p['bit_idx']], np.int64)
    np.savez_compressed(os.path.join(HERE, 'ref_model_io.npz'), X=X.numpy(), y_ref_fp32=y.numpy(),
                        fc1_weight=W1.numpy(), **flat)
    print('wrote', out, os.path.getsize(out), 'bytes')


if __name__ == '__main__':
    main()
