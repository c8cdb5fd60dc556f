"""Checkpoint loading at the reference's model dimensions (hs 2560, moe_is 640): a
synthetic sharded .safetensors checkpoint with the ModelOpt tensor names is read through
the C++ io::WeightLoader / LoadMoEWeights shims.  CPU: the packed device layout the loader
produces equals the layout computed independently here (oracle swizzle); contract
violations give the reference's messages.  GPU: the layer loaded from the checkpoint gives,
through MoEForward in C++, the same bits as the Python binding on the same weights."""
import json
import os
import struct
import subprocess

import numpy as np
import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "loader_test")
E, HS, IS, SIS, LAYER = 6, 2560, 640, 640, 3


def _build():
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    pkg = os.path.join(ROOT, "qwen4-thor_b200")
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-pthread", f"-I{cuda}/include", f"-I{ROOT}/include", f"-I{pkg}/host",
           os.path.join(ROOT, "tests", "cpp", "loader_test.cpp"), "-o", EXE,
           f"-L{pkg}", "-lq4t_moe_b200", f"-Wl,-rpath,{pkg}", f"-L{cuda}/lib64", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def write_safetensors(path, tensors):
    """tensors: list of (name, dtype string, shape, bytes)."""
    header, off = {"__metadata__": {"format": "pt"}}, 0
    for name, dtype, shape, data in tensors:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(data)]}
        off += len(data)
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, _, _, data in tensors:
            f.write(data)


def make_checkpoint(directory, seed=11, break_tensor=None):
    """Raw ModelOpt-style tensors of one layer, spread over two shards; returns the arrays."""
    rng = np.random.default_rng(seed)
    raw = {"experts": []}
    shards = [[], []]
    weight_map = {}
    prefix = f"model.language_model.layers.{LAYER}.mlp"

    def add(shard, name, dtype, shape, data):
        if break_tensor and name.endswith(break_tensor[0]):
            if break_tensor[1] == "drop":
                return
            dtype, shape = break_tensor[1], break_tensor[2] or shape
        shards[shard].append((name, dtype, shape, data))
        weight_map[name] = f"model-{shard + 1:05d}-of-00002.safetensors"

    for e in range(E):
        ex = {}
        for proj, rows, cols in (("gate_proj", IS, HS), ("up_proj", IS, HS), ("down_proj", HS, IS)):
            w = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
            s = rng.integers(40, 64, (rows, cols // 16), dtype=np.uint8)   # benign E4M3 codes
            ws2 = np.float32(0.0005 + 0.0001 * rng.random())
            ins = np.float32(0.0019)
            ex[proj] = (w, s, ws2, ins)
            base = f"{prefix}.experts.{e}.{proj}"
            add(e % 2, base + ".weight", "U8", w.shape, w.tobytes())
            add(e % 2, base + ".weight_scale", "F8_E4M3", s.shape, s.tobytes())
            # a scalar may be rank 0 or a one-element vector
            add(e % 2, base + ".weight_scale_2", "F32", [] if e % 3 else [1], ws2.tobytes())
            add((e + 1) % 2, base + ".input_scale", "F32", [], ins.tobytes())
        raw["experts"].append(ex)
    for name, shape in ((".gate.weight", (E, HS)), (".shared_expert.gate_proj.weight", (SIS, HS)),
                        (".shared_expert.up_proj.weight", (SIS, HS)), (".shared_expert.down_proj.weight", (HS, SIS)),
                        (".shared_expert_gate.weight", (1, HS))):
        a = O.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
        raw[name] = a
        add(1, prefix + name, "BF16", shape, a.tobytes())
    for i in range(2):
        write_safetensors(os.path.join(directory, f"model-{i + 1:05d}-of-00002.safetensors"), shards[i])
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": sum(len(t[3]) for s in shards for t in s)}, "weight_map": weight_map}, f)
    return raw


def expected_layout(raw):
    gu_p, gu_sf, dn_p, dn_sf = [], [], [], []
    for ex in raw["experts"]:
        gu_p.append(np.concatenate([ex["gate_proj"][0], ex["up_proj"][0]]))
        gu_sf.append(O.swizzle_sf(np.concatenate([ex["gate_proj"][1], ex["up_proj"][1]]), 2 * IS, HS))
        dn_p.append(ex["down_proj"][0])
        dn_sf.append(O.swizzle_sf(ex["down_proj"][1], HS, IS))
    scal = [np.array([ex[p][j] for ex in raw["experts"]], np.float32)
            for p, j in (("gate_proj", 2), ("gate_proj", 3), ("down_proj", 2), ("down_proj", 3))]
    return (np.concatenate(gu_p), np.concatenate([s.ravel() for s in gu_sf]), np.concatenate(dn_p),
            np.concatenate([s.ravel() for s in dn_sf]), scal)


def test_loader_packs_reference_dims(q4t, tmp_path):
    if not os.path.exists(q4t.LIB_PATH):
        pytest.skip("library not built")
    _build()
    raw = make_checkpoint(str(tmp_path))
    r = subprocess.run([EXE, "check", str(tmp_path), str(LAYER), str(E), str(HS), str(IS)], capture_output=True, text=True)
    assert r.stdout.startswith("ok shards=2"), r.stdout + r.stderr
    out = tmp_path / "packed.bin"
    r = subprocess.run([EXE, "host", str(tmp_path), str(LAYER), str(E), str(HS), str(IS), str(out)],
                       capture_output=True, text=True)
    assert "host PASS" in r.stdout, r.stdout + r.stderr
    gu_p, gu_sf, dn_p, dn_sf, scal = expected_layout(raw)
    blob = np.fromfile(out, np.uint8)
    pos = 0
    for want in (gu_p, gu_sf, dn_p, dn_sf):
        got = blob[pos:pos + want.size]
        assert np.array_equal(got, want.ravel())
        pos += want.size
    got_scal = blob[pos:].view(np.float32).reshape(4, E)
    for j in range(4):
        assert np.array_equal(got_scal[j], scal[j])


@pytest.mark.parametrize("broken,message", [
    (("experts.2.up_proj.weight", "drop", None), "missing MoE tensor: model.language_model.layers.3.mlp.experts.2.up_proj.weight"),
    (("experts.1.down_proj.weight_scale", "U8", None), "MoE tensor dtype/shape/size mismatch: model.language_model.layers.3.mlp.experts.1.down_proj.weight_scale"),
    (("experts.0.gate_proj.weight", "U8", (IS // 2, HS)), "MoE tensor dtype/shape/size mismatch: model.language_model.layers.3.mlp.experts.0.gate_proj.weight"),
    (("experts.4.gate_proj.input_scale", "F32", (1, 1)), "MoE scalar dtype/shape/size mismatch: model.language_model.layers.3.mlp.experts.4.gate_proj.input_scale"),
])
def test_loader_contract_messages(q4t, tmp_path, broken, message):
    if not os.path.exists(q4t.LIB_PATH):
        pytest.skip("library not built")
    _build()
    make_checkpoint(str(tmp_path), break_tensor=broken)
    r = subprocess.run([EXE, "check", str(tmp_path), str(LAYER), str(E), str(HS), str(IS)], capture_output=True, text=True)
    assert r.stdout.strip() == message, r.stdout + r.stderr


@pytest.mark.gpu
def test_checkpoint_layer_runs_like_the_binding(q4t, gpu_lib, tmp_path):
    import torch
    _build()
    raw = make_checkpoint(str(tmp_path))
    T, k = 5, 2
    x = O.f32_to_bf16(np.random.default_rng(4).standard_normal((T, HS), dtype=np.float32))
    x.tofile(tmp_path / "x.bin")
    r = subprocess.run([EXE, "device", str(tmp_path), str(LAYER), str(E), str(HS), str(IS), str(SIS), str(T), str(k),
                        str(tmp_path / "x.bin"), str(tmp_path / "y.bin")], capture_output=True, text=True, timeout=300)
    assert "device PASS" in r.stdout, r.stdout + r.stderr
    y_cpp = np.fromfile(tmp_path / "y.bin", np.uint16).reshape(T, HS)
    gu_p, gu_sf, dn_p, dn_sf, scal = expected_layout(raw)
    prefix_free = {n: raw[n] for n in raw if n != "experts"}
    L = O.Layer(E, HS, IS, SIS, gu_packed=gu_p, gu_sf=gu_sf, dn_packed=dn_p, dn_sf=dn_sf, gu_w_scale2=scal[0],
                gu_input_scale=scal[1], dn_w_scale2=scal[2], dn_input_scale=scal[3], gate=prefix_free[".gate.weight"],
                shared_gu=np.concatenate([prefix_free[".shared_expert.gate_proj.weight"],
                                          prefix_free[".shared_expert.up_proj.weight"]]),
                shared_down=prefix_free[".shared_expert.down_proj.weight"],
                shared_gate_scalar=prefix_free[".shared_expert_gate.weight"].reshape(-1))
    dl = q4t.DeviceLayer.from_host(L)
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    y = torch.empty((T, HS), dtype=torch.bfloat16, device="cuda")
    fwd = q4t.MoEForward(dl, T, k)
    fwd(xd, y)
    fwd.status()
    assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), y_cpp)
