"""The build variant with time stamps inside its kernels (csrc/trace.cuh, library bf16_trace): it has to be chosen
before the plain library is loaded, so the check runs in a process of its own.  The traced kernels must compute what
the plain ones compute, and their records must be time lines: start <= dependency <= ... <= end."""

import json
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

SCRIPT = textwrap.dedent("""
    import json, math, sys
    import torch
    sys.path.insert(0, sys.argv[1])
    from libmir_b200 import kernels
    kernels.use_traced_kernels()
    torch.manual_seed(0)
    rows, n, k = 8, 512, 1024
    x = (torch.randn(rows, k, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
    out = torch.empty(rows, n, device="cuda", dtype=torch.bfloat16)
    kernels.stream_linear(x, w, out)
    want = x.float() @ w.float().t()
    product_error = float((out.float() - want).abs().max())
    # decode attention over two requests (tcgen05 kernel, two partitions, the merge for few partitions)
    heads, kv_heads, dim, page, lengths = 8, 2, 128, 16, [300, 40]
    pages = [-(-length // page) for length in lengths]
    pool_rows = (sum(pages) + 2) * page
    k_pool = torch.randn(pool_rows, kv_heads, dim, device="cuda").bfloat16()
    v_pool = torch.randn(pool_rows, kv_heads, dim, device="cuda").bfloat16()
    table = torch.full((2, max(pages)), -1, dtype=torch.int32, device="cuda")
    cursor = 0
    for r, count in enumerate(pages):
        table[r, :count] = torch.arange(cursor, cursor + count, dtype=torch.int32)
        cursor += count
    positions = torch.tensor([length - 1 for length in lengths], dtype=torch.int32, device="cuda")
    qkv = torch.randn(2, (heads + 2 * kv_heads) * dim, device="cuda").bfloat16()
    attended = torch.empty(2, heads * dim, device="cuda", dtype=torch.bfloat16)
    partition, count = 256, 2
    scratch = torch.empty(kernels.decode_attention_scratch_floats(2, heads, dim, count), device="cuda")
    scale = 1.0 / math.sqrt(dim)
    kernels.decode_attention(qkv, attended, k_pool, v_pool, table, positions, page, heads, kv_heads, dim, scale, None,
                             partition, count, scratch)
    attention_error = 0.0
    for r, length in enumerate(lengths):
        rows_of = torch.cat([torch.arange(int(p) * page, int(p) * page + page) for p in table[r, :pages[r]]])[:length]
        keys, values = k_pool[rows_of.cuda()].float(), v_pool[rows_of.cuda()].float()
        q = qkv[r, :heads * dim].float().view(heads, dim)
        for h in range(heads):
            weights = torch.softmax(keys[:, h // (heads // kv_heads)] @ q[h] * scale, dim=0)
            expected = weights @ values[:, h // (heads // kv_heads)]
            got = attended[r].float().view(heads, dim)[h]
            attention_error = max(attention_error, float((got - expected).abs().max()))
    # prompt attention over 700 tokens of one request (tcgen05 kernel): the first CTA's tiles
    n = 700
    k_pool = torch.randn(704, kv_heads, dim, device="cuda").bfloat16()
    v_pool = torch.randn(704, kv_heads, dim, device="cuda").bfloat16()
    prompt_table = torch.arange(44, dtype=torch.int32, device="cuda").view(1, 44)
    packed = torch.randn(n, (heads + 2 * kv_heads) * dim, device="cuda").bfloat16()
    prompt_out = torch.empty(n, heads * dim, device="cuda", dtype=torch.bfloat16)
    kernels.prefill_attention(packed, prompt_out, k_pool, v_pool, prompt_table,
                              torch.tensor([0, n], dtype=torch.int32, device="cuda"),
                              torch.tensor([n], dtype=torch.int32, device="cuda"), page, heads, kv_heads, dim, scale, None,
                              tensor_cores=True)
    keys, values = k_pool[:n].float(), v_pool[:n].float()
    prompt_error = 0.0
    for row in (0, 127, 128, 699):
        for h in range(heads):
            weights = torch.softmax(keys[:row + 1, h // (heads // kv_heads)] @ packed[row, h * dim:(h + 1) * dim].float() * scale, dim=0)
            expected = weights @ values[:row + 1, h // (heads // kv_heads)]
            prompt_error = max(prompt_error, float((prompt_out[row].float().view(heads, dim)[h] - expected).abs().max()))
    tiles = kernels.read_prompt_attention_trace()
    records = {name: table_.tolist() for name, table_ in kernels.read_trace().items()}
    print(json.dumps({"product_error": product_error, "attention_error": attention_error, "records": records,
                      "prompt_error": prompt_error, "prompt_tiles": tiles[:8].tolist(), "prompt_items": tiles[200:202].tolist(),
                      "prompt_flag": kernels.prefill_attention_error(),
                      "library": kernels.library("bf16")._name, "flags": [kernels.stream_linear_error(),
                                                                           kernels.decode_attention_error()]}))
""")


def test_traced_kernels_compute_the_same_and_leave_time_lines():
    done = subprocess.run([sys.executable, "-c", SCRIPT, str(ROOT)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert "bf16_trace" in report["library"]
    assert report["flags"] == [0, 0]
    assert report["product_error"] < 0.05 and report["attention_error"] < 0.03
    assert report["prompt_error"] < 0.03 and report["prompt_flag"] == 0
    first = report["prompt_tiles"][0]                           # the first CTA's first tile: its item has six
    # keys asked for <= the issuer has them <= scores issued; the softmax has the scores <= has read them <= knows the
    # maximum <= has the exponentials <= has arrived; then the issuer has P and issues the product with V
    for line in ([first[i] for i in (0, 12, 2)], [first[i] for i in (6, 7, 8, 9, 10)], [first[i] for i in (4, 14)]):
        assert all(stamp > 0 for stamp in line) and all(a <= b for a, b in zip(line, line[1:])), first
    assert first[10] <= first[4] + 2000 and first[2] <= first[6]
    item = report["prompt_items"][0]                            # the end of its first item, in order
    assert all(a <= b for a, b in zip(item[:5], item[1:5])) and item[0] > 0, item
    records = report["records"]
    assert len(records["stream"]) == 2 and len(records["merge"]) >= 1 and len(records["decode"]) >= 1
    assert records["rope"] == []                                # (no such kernel ran)
    for name in ("stream", "decode", "merge"):
        for record in records[name]:
            stamps = [t for t in record[:14] if t > 0]
            assert len(stamps) >= 3 and record[0] > 0, (name, record)
            assert max(stamps) - min(stamps) < 50_000_000, (name, record)     # within 50 ms of each other
    for record in records["stream"]:                            # start <= dependency <= ... <= second barrier
        line = [record[i] for i in (0, 2, 4, 6, 7, 8, 9)]
        assert all(a <= b for a, b in zip(line, line[1:])), record
    for record in records["decode"]:                            # set up <= first scores <= ... <= end
        line = [record[i] for i in (1, 6, 7, 10, 11, 12)]
        assert all(a <= b for a, b in zip(line, line[1:])), record
        assert record[14] in (1, 2)                              # tiles of the traced CTAs
