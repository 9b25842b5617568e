"""Generates the golden vectors in this directory by running the REFERENCE's own native module
(``oracle/_ref/_C.so``, built from its unmodified sources by ``oracle/build_ref.py``) on small seeded inputs.

Needs a GPU:  python tests/golden/make_golden.py <output-dir>
The committed ``reference_vectors.npz`` is the output of this script on a B200; ``tests/test_golden.py`` checks the
CPU oracle against it on machines without a GPU.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]


def load_reference():
    spec = importlib.util.spec_from_file_location("_C", str(ROOT / "oracle" / "_ref" / "_C.so"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def padded(t):
    big = torch.zeros(t.shape[0] + 64, dtype=t.dtype, device=t.device)
    big[:t.shape[0]] = t
    return big[:t.shape[0]]


def main(out_dir):
    ref = load_reference()
    rng = np.random.default_rng(2026)
    # a wavy sheet + a random blob, shifted by a 32-voxel margin
    n = 1500
    x, y = rng.uniform(0, 40, n), rng.uniform(0, 40, n)
    sheet = np.stack([x, y, 12 + 4 * np.sin(x / 5) + 3 * np.cos(y / 4)], 1)
    blob = rng.uniform(10, 18, size=(500, 3))
    coords = np.unique(np.floor(np.concatenate([sheet, blob])).astype(np.int32) + 32, axis=0)
    coords = coords[rng.permutation(len(coords))]
    out = {"coords": coords}
    c = torch.from_numpy(coords).cuda()
    for double in (False, True):
        tag = "u64" if double else "u32"
        keys, perm = ref.cuda_flatten_sort(c, double)
        out[f"{tag}_keys"], out[f"{tag}_perm"] = keys.cpu().numpy(), perm.cpu().numpy()
        out[f"{tag}_unflat"] = ref.cuda_unflatten(keys).cpu().numpy()
        strides = [(2, 2, 2), (4, 4, 4), (8, 8, 16)]
        levels = ref.cuda_streamed_output_generate(keys, strides)
        for s, lv in zip(strides, levels):
            out[f"{tag}_down_{s[0]}_{s[1]}_{s[2]}"] = lv.cpu().numpy()
        src = padded(keys)
        cases = [("sub3", src, src, (3, 3, 3), (1, 1, 1)), ("sub5", src, src, (5, 5, 5), (1, 1, 1)),
                 ("down3", src, levels[0], (3, 3, 3), (1, 1, 1)), ("down2", src, levels[0], (2, 2, 2), (1, 1, 1)),
                 ("lvl2", padded(levels[0]), levels[1], (3, 3, 3), (2, 2, 2))]
        for name, s_, t_, ks, st in cases:
            m0 = ref.cuda_binary_search(s_, t_, ks, st, 0)
            m1 = ref.cuda_binary_search(s_, t_, ks, st, 1)
            out[f"{tag}_{name}_os"] = m0[2].cpu().numpy()
            out[f"{tag}_{name}_ws"] = m1[2].cpu().numpy()
            out[f"{tag}_{name}_nbmaps"] = m1[3].cpu().numpy()
            out[f"{tag}_{name}_nbsizes"] = m1[4].cpu().numpy()
            out[f"{tag}_{name}_naddrs"] = m1[5].cpu().numpy()
            out[f"{tag}_{name}_qnaddrs"] = m1[6].cpu().numpy()
            out[f"{tag}_{name}_sizes"] = np.array([m1[7], m1[8]], dtype=np.int32)
            if name == "down3":
                out[f"{tag}_{name}_inverse"] = ref.cuda_convert_transposed_os(m0[2], s_.shape[0]).cpu().numpy()
                m2 = ref.cuda_binary_search(s_, t_, ks, st, 2)
                out[f"{tag}_{name}_smask"] = m2[3].cpu().numpy()
                out[f"{tag}_{name}_tmask"] = m2[4].cpu().numpy()
            if name in ("sub3", "sub5"):
                # the submanifold mask format (mirrored halves) and the hybrid dataflows: every slot of the 9-tuple
                for df in range(2, 9):
                    m = ref.cuda_binary_search(s_, t_, ks, st, df)
                    out[f"{tag}_{name}_df{df}_map"] = m[2].cpu().numpy()
                    for slot in (3, 4, 5, 6):
                        if m[slot] is not None:
                            out[f"{tag}_{name}_df{df}_slot{slot}"] = m[slot].cpu().numpy()
                    if m[7] is not None:
                        out[f"{tag}_{name}_df{df}_sizes"] = np.array([m[7], m[8]], dtype=np.int32)
            if name == "sub3" and not double:
                nsrc = s_.shape[0]
                feats = torch.from_numpy(rng.normal(size=(nsrc, 16)).astype(np.float16)).cuda()
                w = torch.from_numpy((rng.normal(size=(27, 16, 16)) / np.sqrt(27 * 16)).astype(np.float16)).cuda()
                out["feats"], out["weights"] = feats.cpu().numpy(), w.cpu().numpy()
                out["conv_os_on_os_map"] = ref.cuda_sparse_convolution_forward_os(nsrc, nsrc, m0[2], feats, w).cpu().numpy()
                out["conv_ws_merged"] = ref.cuda_sparse_convolution_forward_ws_merged(
                    nsrc, nsrc, feats, w, m1[5], m1[6], m1[3], m1[7], m1[8], False).cpu().numpy()
                # mask-format and hybrid forward calls on the same features and kernel tensor (each dataflow reads the
                # kernel tensor in its own offset order)
                for df in range(2, 9):
                    m = ref.cuda_binary_search(s_, t_, ks, st, df)
                    if df == 2:
                        y = ref.cuda_sparse_convolution_forward_ws(nsrc, nsrc, 16, 16, 4, -1, feats, w, m[3], m[4], m[5])
                    elif df % 2 == 1:
                        y = ref.cuda_sparse_convolution_forward_hs_merged(nsrc, nsrc, feats, w, m[5], m[6], m[3],
                                                                          None if df == 3 else m[2], m[7], m[8], False)
                    else:
                        y = ref.cuda_sparse_convolution_forward_hs(nsrc, nsrc, 16, 16, 4, -1, feats, w, m[3], m[4], m[5],
                                                                   None if df == 4 else m[2])
                    out[f"conv_df{df}"] = y.cpu().numpy()
    torch.cuda.synchronize()
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    np.savez_compressed(Path(out_dir) / "reference_vectors.npz", **out)
    print("wrote", Path(out_dir) / "reference_vectors.npz", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).resolve().parent))
