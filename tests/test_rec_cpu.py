"""Fixed-step beam generation (generative recommendation) on the tiny CPU model: the batched engine with
x-attention over shared prompt pages returns the same items and scores as an exhaustive recomputation,
with and without a catalogue of valid items, and leaks no KV block."""
import torch

from xllm_b200 import LLM
from xllm_b200.engine.rec import ItemTrie, RecEngine, recommend_reference
from xllm_b200.ops import xattn


def _llm():
    return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=128, max_seqs_per_batch=8,
               max_tokens_per_batch=256, enable_graph=False, enable_prefix_cache=False)


def test_xattention_reference_matches_dense_attention():
    g = torch.Generator().manual_seed(0)
    nq, nkv, d, page, cap = 4, 2, 32, 16, 2
    lens, W = [21, 40], 3
    nb = 8
    kc, vc = torch.randn(nb, nkv, page, d, generator=g), torch.randn(nb, nkv, page, d, generator=g)
    bt = torch.tensor([[1, 2, 0], [3, 4, 5]], dtype=torch.int32)
    rows = len(lens) * W
    q = torch.randn(rows, nq, d, generator=g)
    ku, vu = torch.randn(rows, nkv, cap, d, generator=g), torch.randn(rows, nkv, cap, d, generator=g)
    anc = torch.stack([torch.tensor([1, 0, 0, 5, 5, 3]), torch.arange(rows)]).to(torch.int32)
    cu = torch.tensor([0, W, 2 * W], dtype=torch.int32)
    out = xattn.xattention(q, kc, vc, bt, cu, torch.tensor(lens, dtype=torch.int32), W, ku, vu, anc, 2, 0.2)
    for row in range(rows):
        b = row // W
        blocks = bt[b, : (lens[b] + page - 1) // page].long()
        k = kc[blocks].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, : lens[b]]
        v = vc[blocks].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, : lens[b]]
        k = torch.cat([k, ku[int(anc[0, row]), :, 0][:, None], ku[row, :, 1][:, None]], 1).repeat_interleave(nq // nkv, 0)
        v = torch.cat([v, vu[int(anc[0, row]), :, 0][:, None], vu[row, :, 1][:, None]], 1).repeat_interleave(nq // nkv, 0)
        p = torch.softmax(torch.einsum("hd,hkd->hk", q[row], k) * 0.2, -1)
        assert torch.allclose(out[row], torch.einsum("hk,hkd->hd", p, v), atol=1e-5)


def test_rec_engine_matches_exhaustive_beam():
    llm = _llm()
    rec = RecEngine(llm.engine)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (19, 33, 8)]
    got = rec.generate(prompts, beam_width=4, num_steps=3)
    assert len(got) == 3
    for p, items in zip(prompts, got):
        want = recommend_reference(llm.engine, p, 4, 3)
        assert [it.token_ids for it in items] == [w.token_ids for w in want]
        for a, b in zip(items, want):
            assert abs(a.logprob - b.logprob) < 1e-3
        assert all(items[i].logprob >= items[i + 1].logprob for i in range(len(items) - 1))
    assert llm.engine.scheduler.block_manager(0).num_used_blocks == 0


def test_rec_engine_respects_the_catalogue():
    llm = _llm()
    rec = RecEngine(llm.engine)
    g = torch.Generator().manual_seed(9)
    V = llm.engine.args.vocab_size
    items = [tuple(torch.randint(0, V, (3,), generator=g).tolist()) for _ in range(40)]
    items += [(items[0][0], items[0][1], 5), (items[0][0], 17, 9)]          # shared prefixes
    trie = ItemTrie(items, V)
    prompt = torch.randint(0, V, (25,), generator=g).tolist()
    got = rec.generate([prompt], beam_width=8, num_steps=3, trie=trie)[0]
    assert len(got) == 8 and all(tuple(it.token_ids) in set(items) for it in got)
    want = recommend_reference(llm.engine, prompt, 8, 3, trie=trie)
    assert [it.token_ids for it in got] == [w.token_ids for w in want]
    # a beam wider than the catalogue returns the whole catalogue and nothing else
    small = ItemTrie(items[:5], V)
    got = rec.generate([prompt], beam_width=16, num_steps=3, trie=small)[0]
    assert sorted(tuple(it.token_ids) for it in got) == sorted(set(items[:5]))
    assert llm.engine.scheduler.block_manager(0).num_used_blocks == 0


def test_rec_backend_over_http_and_offline_api():
    import http.client
    import json
    import threading

    from xllm_b200.api.server import ApiServer
    llm = _llm()
    prompt = list(range(100, 130))
    offline = llm.recommend([prompt], beam_width=5, num_steps=3)[0]
    srv = ApiServer(llm.engine, None, model_name="tiny-rec", host="127.0.0.1", port=0, backend="rec")
    t = threading.Thread(target=srv.serve_forever, args=(10,), daemon=True)
    t.start()
    try:
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
        c.request("POST", "/v1/completions", json.dumps({"prompt": prompt, "beam_width": 5, "max_tokens": 3}),
                  {"Content-Type": "application/json"})
        r = c.getresponse()
        obj = json.loads(r.read().decode())
        assert r.status == 200 and len(obj["choices"]) == 5
        assert [ch["token_ids"] for ch in obj["choices"]] == [it.token_ids for it in offline]
        assert obj["usage"]["completion_tokens"] == 15
        items = [ch["token_ids"] for ch in obj["choices"][:3]]
        c.request("POST", "/v1/completions", json.dumps({"prompt": prompt, "beam_width": 8, "max_tokens": 3,
                                                         "valid_items": items}), {"Content-Type": "application/json"})
        r = c.getresponse()
        obj = json.loads(r.read().decode())
        assert r.status == 200 and sorted(ch["token_ids"] for ch in obj["choices"]) == sorted(items)
        c.request("POST", "/v1/completions", json.dumps({"prompt": prompt, "max_tokens": 99}),
                  {"Content-Type": "application/json"})
        r = c.getresponse()
        r.read()
        assert r.status == 400
        c.close()
    finally:
        srv.shutdown()
        t.join(timeout=5)


def test_item_trie_masks_and_node_ids_match_brute_force():
    """The CSR trie's masks and node transitions against sets built by hand, for a random catalogue with
    shared prefixes, duplicates and beams that leave the catalogue."""
    g = torch.Generator().manual_seed(5)
    V, depth = 97, 3
    items = torch.randint(0, 12, (400, depth), generator=g).tolist() + torch.randint(0, V, (300, depth), generator=g).tolist()
    trie = ItemTrie(items + items[:50], V)
    assert trie.n_items == len({tuple(i) for i in items}) and trie.depth == depth
    cat = {tuple(i) for i in items}
    assert tuple(items[3]) in trie
    assert ((96, 96, 96) in trie) == ((96, 96, 96) in cat)
    rows = 64
    prefixes = [tuple(items[i][:0]) for i in range(rows)]
    nodes = trie.root(rows)
    for level in range(depth):
        mask = trie.mask_of(level, nodes)
        for r, pre in enumerate(prefixes):
            want = {it[level] for it in cat if it[:level] == pre} if pre is not None else set()
            assert set(mask[r].nonzero().flatten().tolist()) == want, (level, r)
        # half the rows follow an item, a quarter take a random token, a quarter are already dead
        nxt = []
        for r, pre in enumerate(prefixes):
            if pre is not None and r % 4 != 3:
                nxt.append(items[(r * 7) % len(items)][level] if items[(r * 7) % len(items)][:level] == list(pre) else
                           next(iter(sorted(it[level] for it in cat if it[:level] == pre))))
            else:
                nxt.append(int(torch.randint(0, V, (1,), generator=g)))
        nodes = trie.advance(level, nodes, torch.tensor(nxt))
        new_prefixes = []
        for r, pre in enumerate(prefixes):
            p = None if pre is None else pre + (nxt[r],)
            if p is not None and not any(it[:level + 1] == p for it in cat):
                p = None
            new_prefixes.append(p)
            assert (int(nodes[r]) >= 0) == (p is not None), (level, r)
        prefixes = new_prefixes
    assert any(p is None for p in prefixes) and any(p is not None for p in prefixes)
    assert torch.equal(trie.allowed([tuple(items[0][:2]), tuple(items[1][:2])], "cpu"),
                       torch.stack([torch.tensor([any(it[:2] == tuple(items[j][:2]) and it[2] == v for it in cat) for v in range(V)])
                                    for j in (0, 1)]))
