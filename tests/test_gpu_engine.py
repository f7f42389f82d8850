"""The batch engine as a decode engine: eight sequences with different histories decode 300
tokens through BatchEngine.decode_step (batched pre-step, batched compression events, re-planned
batched attention) and must end in the state, and produce the outputs, of eight independent
single-sequence runtimes (KhqRuntime, the host state machine of src/khq/runtime.mojo:454-613)
fed the same projections."""
import numpy as np
import pytest

import cases
from cases import D, H_KV, H_Q, SCALE

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("generation", [2, 3, 4])
def test_engine_decodes_like_independent_runtimes(cuda_ops, generation):
    import torch

    from bonsai_mojo_1bit_optimization_t4_cuda_b200.engine import BatchEngine
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.runtime import KhqRuntime

    B, steps = 8, 300
    layer_ids = [3, 7]
    rng = np.random.default_rng(2027)
    sk, sv = cases.synth.channel_scales(rng), cases.synth.channel_scales(rng)
    sample_k, sample_v = cases.synth.make_kv(rng, 128, sk, sv)
    tables = [cases.synth.make_tables(rng, li, sample_k.reshape(-1, D), sample_v.reshape(-1, D), vq_scale=1.0 / 16.0)
              for li in layer_ids]
    norm_w = [((1 + 0.1 * rng.standard_normal(D)).astype(np.float32), (1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
              for _ in layer_ids]
    start = [0, 17, 17, 40, 63, 90, 127, 200]  # raw tokens each sequence already holds; two share a history length

    def projections(step, seq, layer):
        g = np.random.default_rng([step + 100_000, seq, layer])
        q = g.standard_normal((H_Q, 2 * D)).astype(np.float16)
        k = (g.standard_normal((H_KV, D)) * sk).astype(np.float16)
        v = (g.standard_normal((H_KV, D)) * sv).astype(np.float16)
        return q, k, v

    # ---- reference: one runtime per sequence ------------------------------------------------------
    rts = []
    for s in range(B):
        rt = KhqRuntime(cuda_ops, device="cuda")
        assert rt.khq_activate(tables, max_seq=1024)
        for li in layer_ids:
            rt.khq_init_layer(li, H_Q, H_KV, D)
        rts.append(rt)

    def runtime_step(rt, seq, step_id, pos):
        outs = []
        for l, li in enumerate(layer_ids):
            q, k, v = projections(step_id, seq, l)
            qg, kd, vd = torch.from_numpy(q).cuda().reshape(-1), torch.from_numpy(k).cuda().reshape(-1), torch.from_numpy(v).cuda().reshape(-1)
            out = torch.zeros(H_Q * D, dtype=torch.float16, device="cuda")
            assert rt.khq_prestep(li, qg, kd, vd, pos, torch.from_numpy(norm_w[l][0]).cuda(), torch.from_numpy(norm_w[l][1]).cuda())
            assert rt.khq_step(li, qg, kd, vd, out, SCALE, rings_written=True)
            outs.append(out)
        return outs

    for s in range(B):  # histories: negative step ids so that they never collide with the common steps
        for t in range(start[s]):
            runtime_step(rts[s], s, -1 - t, t)
    # ---- the engine starts from those histories ------------------------------------------------------
    eng = BatchEngine(tables, [0] * B, start, device="cuda", codebook_in_smem=generation, grow_tokens=512, norm_weights=norm_w)
    for l, li in enumerate(layer_ids):
        for s in range(B):
            if start[s]:
                T = rts[s].layers[li].t
                n = start[s] * H_KV * D
                eng.load_window(l, s, T["ring_k"][:n], T["ring_v"][:n], T["ring_u"][:n])
    worst = 0.0
    for step in range(steps):
        for l in range(len(layer_ids)):
            for s in range(B):
                q, k, v = projections(step, s, l)
                eng.h_q[l, s].copy_(torch.from_numpy(q).reshape(-1))
                eng.h_k[l, s].copy_(torch.from_numpy(k).reshape(-1))
                eng.h_v[l, s].copy_(torch.from_numpy(v).reshape(-1))
        out = eng.decode_step(SCALE)
        torch.cuda.synchronize()
        got = out.float().numpy().reshape(len(layer_ids), B, H_Q, D).copy()
        check_outputs = step < 4 or step % 16 == 0 or step >= steps - 2 or any((start[s] + step + 1) in (255, 256, 257) for s in range(B))
        for s in range(B):
            want = runtime_step(rts[s], s, step, start[s] + step)
            if check_outputs:
                torch.cuda.synchronize()
                for l in range(len(layer_ids)):
                    ok, mx, exc = cases.attention_close(got[l, s], want[l].float().cpu().numpy().reshape(H_Q, D))
                    worst = max(worst, mx)
                    assert ok, f"step {step} sequence {s} layer {l}: max abs {mx:.3e} excess {exc:.3e}"
    assert cuda_ops.lib.khq_b200_device_status() == 0
    # ---- final state: positions, code words of every compressed token, raw rings ---------------------
    assert eng.events_fired == sum(1 for s in range(B) if start[s] + steps >= 256) + sum(1 for s in range(B) if start[s] + steps >= 384)
    per_row = dict(k_mask=("kmask", 64), k_payload=("kpay", 40), v_payload=("vpay", 104), v_shared_meta=("vsm", 4),
                   k_norms=("knorm", 2), k_r_norms=("krn", 2), v_norms=("vnorm", 2), v_r_norms=("vrn", 2))
    for s in range(B):
        for l, li in enumerate(layer_ids):
            Lr = rts[s].layers[li]
            assert int(eng.boundary[s]) == Lr.boundary and int(eng.write_pos[s]) == Lr.write_pos
            rows = Lr.boundary * H_KV
            r0 = int(eng.row_off[s])
            for key, (rkey, rb) in per_row.items():
                a = eng.pay[l][key].view(torch.uint8)[r0 * rb:(r0 + rows) * rb]
                b = Lr.t[rkey].view(torch.uint8)[:rows * rb]
                assert torch.equal(a, b), f"sequence {s} layer {l}: code words differ in {key}"
            for ring, rkey in ((eng.ring_k, "ring_k"), (eng.ring_v, "ring_v"), (eng.ring_u, "ring_u")):
                assert torch.equal(ring[l][s].reshape(-1), Lr.t[rkey].reshape(-1)), f"sequence {s} layer {l}: {rkey} differs"
    print(f"engine vs independent runtimes, generation {generation}: {eng.events_fired} events, worst output |err| {worst:.2e}")
