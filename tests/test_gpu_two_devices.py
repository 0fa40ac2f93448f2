"""One process, adapters on two devices.  The opt-in to large dynamic shared memory is a per-device
property of every kernel and the adapter makes its own device current inside each call, so a host that
drives several GPUs from one thread needs no set-up of its own.  Local memory only (no peer access).
Skipped on a one-GPU box."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
pkg = importlib.import_module("ferrum-torrens_b200")
from oracle import oracle as o  # noqa: E402


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_handles_on_two_devices_in_one_process():
    lay = pkg.synth.make_layer(808)
    H, I, E, K, SI = lay.hidden, lay.inter, lay.experts, lay.top_k, lay.shared_inter
    banks = o.HostBanks(*lay.banks, slots=E, gu_rows=2 * I, gu_cols=H, dn_rows=H, dn_cols=I)
    ol = o.Layer(H, I, E, K, SI, lay.gate_w, lay.sh_gate_up, lay.sh_down, lay.sh_gate, banks)
    moes = []
    for d in (0, 1):
        m = pkg.B200MoE(d, pkg.ExpertShapes(H, I), E, experts=E, layers=1, top_k=K, shared_inter=SI, max_tokens=320)
        for e in range(E):
            m.load(0, e, e, lay.fields(e))
        moes.append(m)
    # the current device stays where the caller left it
    torch.cuda.set_device(0)
    for tokens in (8, 320):          # decode kernels, then router-wide / grouped GEMM / dense shared expert
        xb = pkg.synth.make_x(40 + tokens, tokens, H)
        want, want_ids, _ = o.moe_block(ol, pkg.synth.bf16_bits_to_f32(xb), threads=o.max_threads())
        for d, m in enumerate(moes):
            dev = torch.device(f"cuda:{d}")
            t16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)
            out = torch.empty((tokens, H), dtype=torch.float32, device=dev)
            ids = torch.empty((tokens, K), dtype=torch.int32, device=dev)
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            m.moe_block(0, t16(xb), t16(lay.gate_w), t16(lay.sh_gate_up), t16(lay.sh_down), t16(lay.sh_gate), out,
                        ids_out=ids, stream=s)
            m.sync_status(stream=s)
            assert torch.cuda.current_device() == 0
            assert np.array_equal(ids.cpu().numpy(), want_ids), (d, tokens)
            rel = np.linalg.norm(out.cpu().numpy() - want) / np.linalg.norm(want)
            assert rel <= 1e-2, (d, tokens, rel)
    for m in moes:
        m.close()
