"""Decode instance of the two-process PD test: a CPU engine behind a DecodeService on a socket.
argv: port, num_blocks, mode ('serve' | 'vanish': exit right after the first adoption | 'pull': serve and ask
for the peer's offline requests while idle)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    port, num_blocks, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.engine.pd_service import Channel, DecodeService, SocketCopy
    eng = LLMEngine(EngineConfig(model="tiny", device="cpu", dtype="float32", block_size=16, num_blocks=num_blocks,
                                 max_seqs_per_batch=8, max_tokens_per_batch=128, enable_graph=False,
                                 enable_prefix_cache=False))
    ch = Channel.connect("127.0.0.1", port)
    svc = DecodeService(eng, ch, SocketCopy(eng.runner), pull_offline=(mode == "pull"), pull_below=2)
    if mode == "vanish":
        while svc.adopted == 0 and not ch.closed:
            svc.step(0.002)
        os._exit(0)             # between steps, nothing in flight: the peer learns it from the socket
    ok = svc.serve(120.0)
    st = eng.scheduler.block_stats(0)
    print(f"PD_DECODE_DONE ok={ok} adopted={svc.adopted} used={st.num_used} reserved={eng.scheduler.num_reserved()} pulls={svc.pulls_sent}", flush=True)


if __name__ == "__main__":
    main()
