"""Records golden vectors from the REFERENCE implementation on a CUDA device.

Imports nano-vllm's own ``nanovllm.layers.attention`` (its Triton ``store_kvcache`` and its
flash-attn calls) from an installed copy of the reference — ``baseline/_ref`` in this repo,
made with ``pip install --no-deps --target baseline/_ref <reference checkout>`` — runs the
seeded cases of cases.py through ``Attention.forward`` / ``store_kvcache`` exactly as the
model runner would (context set with ``set_context``), and writes one .npz per case:
outputs as raw bf16 bits, cache contents as SHA-256 digests, plus a fingerprint of the inputs.

    python tests/golden/make_golden.py [output_dir]        # needs a GPU with flash-attn + triton

The tests never import the reference; they only read the .npz files committed next to this
script.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases as C  # noqa: E402

REF = C.ROOT / "baseline" / "_ref"


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy()


def main(out_dir: Path) -> None:
    sys.path.insert(0, str(REF))
    from nanovllm.layers.attention import Attention, store_kvcache  # the reference module
    from nanovllm.utils.context import reset_context, set_context
    import flash_attn
    import triton

    dev = torch.device("cuda:0")
    out_dir.mkdir(parents=True, exist_ok=True)
    meta = dict(flash_attn=flash_attn.__version__, triton=triton.__version__, torch=torch.__version__,
                gpu=torch.cuda.get_device_name(0))

    for name, (key, value, k_cache, v_cache, slots) in C.store_cases().items():
        kc, vc = k_cache.to(dev), v_cache.to(dev)
        kd = key.to(dev) if key.is_contiguous() else None
        # keep the strided layout on the device too
        n, hkv, d = key.shape
        kv_dev = torch.cat([key.reshape(n, -1), value.reshape(n, -1)], dim=1).to(dev)
        kdev, vdev = (t.view(n, hkv, d) for t in kv_dev.split(hkv * d, dim=-1))
        store_kvcache(kdev, vdev, kc, vc, slots.to(dev))
        torch.cuda.synchronize()
        np.savez(out_dir / f"{name}.npz", k_cache_sha=C.sha(kc.cpu()), v_cache_sha=C.sha(vc.cpu()),
                 inputs=C.input_fingerprint(key, value, k_cache, v_cache, slots), **meta)
        print(name, "ok")

    for name, case in C.decode_cases().items():
        d = case.to(dev)
        B, Hq, Hkv, D = case.geometry
        layer = Attention(Hq, D, case.scale, Hkv)
        layer.k_cache, layer.v_cache = d.k_cache, d.v_cache
        set_context(False, slot_mapping=d.slot_mapping, context_lens=d.context_lens, block_tables=d.block_tables)
        o = layer(d.q.view(B, -1), d.k_new.view(B, -1), d.v_new.view(B, -1))
        reset_context()
        torch.cuda.synchronize()
        np.savez(out_dir / f"{name}.npz", out=bits(o.view(B, Hq, D)), k_cache_sha=C.sha(d.k_cache.cpu()),
                 v_cache_sha=C.sha(d.v_cache.cpu()),
                 inputs=C.input_fingerprint(case.q, case.k_new, case.v_new, case.k_cache, case.v_cache,
                                            case.context_lens, case.block_tables, case.slot_mapping), **meta)
        print(name, "ok")

    for name, case in C.prefill_cases().items():
        d = case.to(dev)
        N, Hq, D = case.q.shape
        Hkv = case.k.shape[1]
        layer = Attention(Hq, D, case.scale, Hkv)
        layer.k_cache, layer.v_cache = d.k_cache, d.v_cache
        set_context(True, d.cu_seqlens_q, d.cu_seqlens_k, case.max_seqlen_q, case.max_seqlen_k, d.slot_mapping,
                    None, d.block_tables)
        o = layer(d.q.view(N, -1), d.k.view(N, -1), d.v.view(N, -1))
        reset_context()
        torch.cuda.synchronize()
        np.savez(out_dir / f"{name}.npz", out=bits(o.view(N, Hq, D)), k_cache_sha=C.sha(d.k_cache.cpu()),
                 v_cache_sha=C.sha(d.v_cache.cpu()),
                 inputs=C.input_fingerprint(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k,
                                            case.slot_mapping, case.block_tables), **meta)
        print(name, "ok")


if __name__ == "__main__":
    main(Path(sys.argv[1]) if len(sys.argv) > 1 else C.GOLDEN_DIR)
