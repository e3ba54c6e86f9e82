"""Child process of tests/test_gpu_serialization.py: load a weight-set file written by another
process, decode it, and print the SHA-256 of every tensor's BF16 bits and its shape as JSON."""
import hashlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(path: str, mapping: str) -> None:
    import torch
    from losslessly_compressed_tensors_b200 import config
    from losslessly_compressed_tensors_b200.operations import decompress
    from losslessly_compressed_tensors_b200.serialization import load_weight_set

    config.lane_mapping = mapping
    compressed = load_weight_set(path)
    batch = load_weight_set(path, decode=True)
    report = {}
    for name, c in compressed.items():
        dense = decompress(c)
        assert torch.equal(dense.view(torch.int16), batch[name].view(torch.int16)), name
        bits = dense.contiguous().view(torch.int16).cpu().numpy().tobytes()
        report[name] = {"sha": hashlib.sha256(bits).hexdigest(), "shape": list(dense.shape),
                        "memory_size": c.memory_size()}
    print(json.dumps(report))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
