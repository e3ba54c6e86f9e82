"""The package under the reference's import name (no GPU needed: imports only)."""
import subprocess
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys
sys.path.insert(0, {root!r})
import losslessly_compressed_tensors_b200.compat as compat
names = compat.install_as_lct()
assert "LCT.operations" in names and "LCT.components.sparse_utils" in names
from LCT.comp_format import Distribution, DistType, NoiseLevel, StorageLayout
from LCT.tensor_buffer import TensorBuffer, Allocation, verify_buffer, visualize_buffer, _free_regions_snapshot
from LCT.comp_tensor import CompressedTensor
from LCT.compression.huffman_tables import FIRST_BITS, FIRST_MASK, get_distribution_tables
from LCT.codec.geometry import geometry
from LCT.components.dist_configs import momentum_dist
from LCT import config
import LCT.operations as ops
import losslessly_compressed_tensors_b200.operations as ours
assert ops is ours and FIRST_BITS == 10 and FIRST_MASK == 1023
for name in ("compress", "decompress", "compA_add_B", "compA_mul_B", "a_compA_add_B",
             "a_compA_add_b_B", "a_compA_add_compB", "A_compB", "A_compBT"):
    assert callable(getattr(ops, name)), name
assert geometry(Distribution(DistType.LAPLACE)) == (65536, 256, 256, 25)
config.lane_mapping = "linear"
import losslessly_compressed_tensors_b200.config as our_config
assert our_config.lane_mapping == "linear"
our_config.check()
config.lane_mapping = "diagonal"
try:
    our_config.check()
    raise SystemExit("bad mapping accepted")
except ValueError:
    pass
print("COMPAT-OK")
"""


def test_package_is_importable_under_the_reference_name():
    out = subprocess.run([sys.executable, "-c", SCRIPT.format(root=ROOT)], capture_output=True,
                         text=True, timeout=300)
    assert out.returncode == 0 and "COMPAT-OK" in out.stdout, out.stdout + out.stderr
