"""The drop-in claim, exercised with the reference's own caller.

``oracle/build_ref_ext.py`` compiles the reference's PyTorch extension
(python/ms_blkq4linear_ext/ms_blkq4linear.cpp) UNCHANGED against this repository's
``include/ms_blkq4gemm.h`` and ``libms_blkq4gemm.so``, the way the reference's
python/setup.py:16-22 links its own library.  This test loads that binary in a fresh process
(this package's own extension carries the same module name) and drives it the way the
reference's ``BlkQ4Linear`` does (python/ms_blkq4linear.py:10-28: ``quant`` in the constructor,
``forward`` + bias per call); where the reference tree is present the reference's Python class
itself is used.  Results are checked against the oracle: packed tensors bit for bit, outputs
within the GEMM tolerance.  Skipped when the binary has not been built."""
import os
import subprocess
import sys
import sysconfig

import pytest

from tests._util import ROOT

pytestmark = pytest.mark.gpu

REF_EXT = os.path.join(ROOT, "oracle", "_ref", "ms_blkq4linear_ext" + sysconfig.get_config_var("EXT_SUFFIX"))

WORKER = r'''
import os, sys
import numpy as np
import torch
root, ref_ext_dir, ref_py_dir = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path.insert(0, ref_ext_dir)
sys.path.insert(0, root)
import ms_blkq4linear_ext as ext                      # the reference's extension, this library underneath
assert os.path.dirname(os.path.abspath(ext.__file__)) == os.path.abspath(ref_ext_dir), ext.__file__
from oracle import blkq4_oracle as O

BlkQ4Linear = None
if ref_py_dir and os.path.exists(os.path.join(ref_py_dir, "ms_blkq4linear.py")):
    sys.path.insert(0, ref_py_dir)
    from ms_blkq4linear import BlkQ4Linear            # the reference's own module


class CallsOfTheReferenceModule:
    """The reference module's call sequence, for boxes without the reference tree."""
    def __init__(self, block_size, col_wise, scale_only, weights, bias_tensor=None):
        self.block_size, self.col_wise, self.has_offsets = block_size, col_wise, not scale_only
        self.in_features, self.out_features = weights.size(1), weights.size(0)
        self.q_weights, self.q_scales, self.q_zp = ext.quant(block_size, col_wise, self.has_offsets, weights)
        self.bias = bias_tensor
    def __call__(self, input):
        output = ext.forward(self.block_size, self.col_wise, self.in_features, self.out_features, input,
                             self.q_weights, self.q_scales, self.q_zp)
        if self.bias is not None:
            output += self.bias
        return output


Layer = BlkQ4Linear or CallsOfTheReferenceModule
g = torch.Generator().manual_seed(0)
for block, col_wise, N, K in [(32, True, 768, 1024), (64, True, 4096, 4096), (16, False, 256, 512), (64, False, 512, 576)]:
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.float16)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.float16).cuda()
    layer = Layer(block, col_wise, False, w.cuda(), bias)
    pw, ps, pz = O.quant_prepack(block, col_wise, w.numpy(), True)
    assert (layer.q_weights.cpu().numpy() == pw).all(), "packed weights differ from the oracle"
    assert (layer.q_scales.cpu().numpy().view(np.uint16) == ps.view(np.uint16)).all(), "scales differ"
    assert (layer.q_zp.cpu().numpy() == pz).all(), "zero points differ"
    wdq = O.dequant(block, col_wise, K, N, pw, ps, pz)
    for M in (1, 16, 300):
        x = torch.randn(M, K, generator=g).to(torch.float16)
        got = layer(x.cuda()).float().cpu().numpy()
        want = O.gemm(x.numpy(), wdq).astype(np.float32) + bias.float().cpu().numpy()
        tol = 1e-2 * np.sqrt(K) * float(x.abs().max()) * float(np.abs(wdq.astype(np.float32)).max())
        err = float(np.abs(got - want).max())
        assert err <= tol, (block, col_wise, M, err, tol)
torch.cuda.synchronize()
print("DROPIN_OK", "reference module" if BlkQ4Linear else "reference extension")
'''


@pytest.mark.skipif(not os.path.exists(REF_EXT), reason="reference extension not built (python oracle/build_ref_ext.py)")
def test_reference_extension_runs_on_this_library(tmp_path):
    ref_py = os.path.join(os.environ.get("BLKQ4_REFERENCE_DIR", os.path.join(ROOT, os.pardir, "reference")), "python")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    r = subprocess.run([sys.executable, str(script), ROOT, os.path.dirname(REF_EXT), ref_py if os.path.isdir(ref_py) else ""],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "DROPIN_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
