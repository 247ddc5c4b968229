"""The metric names of the service, by kind, and the publisher that fills them from the engine.

The catalogue is the reference's (xllm/core/common/metrics.cpp: 116 names; dashboards and alerts
written for it keep working).  `register_all()` creates every series so that `/metrics` exposes the
full set from the first scrape; `EnginePublisher.tick()` is called by the serving loop once per
iteration and costs a few dictionary reads.  Series that belong to parts this engine does not have
(the Mooncake store) stay at zero.
"""
from __future__ import annotations

import os
import time

from .. import _rt

HISTOGRAMS = """end_2_end_latency_milliseconds inter_token_latency_microseconds inter_token_latency_milliseconds
json_object_mask_batch_build_latency_microseconds json_object_mask_device_copy_latency_microseconds
json_object_mask_row_build_latency_microseconds json_object_mask_vocab_scan_latency_microseconds
mooncake_transfer_latency_microseconds_read mooncake_transfer_latency_microseconds_write num_generated_tokens_per_request
num_prompt_tokens_per_request prefix_cache_block_matched_num prefix_cache_block_matched_rate
prepare_input_latency_microseconds rec_first_token_latency_microseconds rec_input_token_num_per_request
rec_sampling_latency_microseconds rec_second_token_latency_microseconds rec_third_token_latency_microseconds
rec_total_latency_microseconds speculative_draft_token_d2h_latency_microseconds time_to_first_token_latency_milliseconds
active_kv_cache_size_in_kilobytes speculative_draft_token_bulk_read_latency_microseconds""".split()

COUNTERS = """allocate_blocks_latency_seconds chat_template_latency_seconds detokenization_latency_seconds_non_stream
detokenization_latency_seconds_stream engine_latency_seconds execution_latency_seconds_logits_processing
execution_latency_seconds_model execution_latency_seconds_sampling json_object_mask_build_calls_draft_total
json_object_mask_build_calls_normal_total json_object_mask_build_calls_target_total
json_object_mask_build_constrained_rows_draft_total json_object_mask_build_constrained_rows_normal_total
json_object_mask_build_constrained_rows_target_total json_object_mask_build_rows_draft_total
json_object_mask_build_rows_normal_total json_object_mask_build_rows_target_total json_object_mask_cache_hits_total
json_object_mask_cache_misses_total mooncake_transfer_bytes_total_read mooncake_transfer_bytes_total_write
mooncake_transfer_completed_total_read mooncake_transfer_completed_total_write mooncake_transfer_failed_total
num_model_execution_total_eager num_processing_tokens_total_generated num_processing_tokens_total_prompt
prefix_cache_latency_seconds_evict prefix_cache_latency_seconds_insert prefix_cache_latency_seconds_match
prefix_cache_match_length_total prepare_input_latency_seconds proto_latency_seconds_i2proto proto_latency_seconds_o2proto
proto_latency_seconds_proto2i proto_latency_seconds_proto2o request_handling_latency_seconds_chat
request_handling_latency_seconds_completion request_status_total_cancelled request_status_total_deadline_exceeded
request_status_total_invalid_argument request_status_total_ok request_status_total_resource_exhausted
request_status_total_unauthenticated request_status_total_unavailable request_status_total_unimplemented
request_status_total_unknown responsing_latency_seconds_non_stream responsing_latency_seconds_stream
scheduling_latency_seconds server_request_in_total server_request_total_fail server_request_total_limit
server_request_total_ok speculative_draft_token_handoff_fallback_total speculative_execution_latency_seconds_draft
speculative_execution_latency_seconds_target speculative_execution_latency_seconds_validation
speculative_num_accepted_tokens_constrained_total speculative_num_accepted_tokens_plain_total
speculative_num_accepted_tokens_total speculative_num_committed_tokens_total
speculative_num_draft_tokens_constrained_total speculative_num_draft_tokens_plain_total speculative_num_draft_tokens_total
speculative_num_drafts_total tokenization_latency_seconds worker_service_latency_seconds
num_generated_tokens_total num_prompt_tokens_total""".split()

GAUGES = """kv_cache_utilization_perc num_blocks_in_prefix_cache num_concurrent_requests num_free_blocks
num_offline_decode_preempt_offline_requests num_online_decode_preempt_offline_requests
num_online_decode_preempt_online_requests num_online_prefill_preempt_offline_requests num_pending_requests
num_preempted_requests num_running_requests num_running_sequences num_used_blocks num_waiting_requests
rec_beam_search_width speculative_mean_tokens_per_decode_step total_activation_size_in_kilobytes
total_kv_cache_size_in_kilobytes total_memory_size_in_kilobytes weight_size_in_kilobytes xllm_cpu_num xllm_cpu_utilization
xllm_gpu_num xllm_gpu_utilization kv_cache_utilization""".split()


def register_all():
    for n in COUNTERS:
        _rt.metric_counter_add(n, 0.0)
    for n in GAUGES:
        _rt.metric_gauge_set(n, _rt.metric_gauge(n))
    # a histogram appears with its first observation; until then it is exposed through a gauge of
    # the same name carrying NaN would be wrong, so histograms are simply listed by `catalog()`


def catalog():
    return {"counter": list(COUNTERS), "gauge": list(GAUGES), "histogram": list(HISTOGRAMS)}


class EnginePublisher:
    """Scheduler, cache, memory and speculative-decoding series of one engine."""

    def __init__(self, engine):
        self.e = engine
        self._last = {}
        self._next_slow = 0.0
        r = engine.runner
        try:
            kv_kb = r.kv_tensor.numel() * r.kv_tensor.element_size() / 1024.0
        except Exception:
            kv_kb = 0.0
        w_kb = sum(t.numel() * t.element_size() for _, t in engine.model.named_params()) / 1024.0
        _rt.metric_gauge_set("total_kv_cache_size_in_kilobytes", kv_kb)
        _rt.metric_gauge_set("weight_size_in_kilobytes", w_kb)
        _rt.metric_gauge_set("xllm_cpu_num", float(os.cpu_count() or 0))

    def _delta(self, key, value):
        d = value - self._last.get(key, 0)
        self._last[key] = value
        return max(d, 0)

    def tick(self, n_calls: int = 0, step_seconds: float = 0.0):
        s = self.e.scheduler
        st = s.block_stats(0)
        g = _rt.metric_gauge_set
        g("num_running_requests", float(s.num_running))
        g("num_running_sequences", float(s.num_running))
        g("num_waiting_requests", float(s.num_waiting))
        g("num_pending_requests", float(s.num_waiting))
        g("num_concurrent_requests", float(n_calls))
        g("num_free_blocks", float(st.num_free))
        g("num_used_blocks", float(st.num_used))
        g("num_blocks_in_prefix_cache", float(st.num_evictable))
        util = float(s.kv_utilization(0))
        g("kv_cache_utilization", util)
        g("kv_cache_utilization_perc", util * 100.0)
        g("num_preempted_requests", float(s.num_preemptions))
        c = _rt.metric_counter_add
        if step_seconds > 0:
            c("engine_latency_seconds", step_seconds)
        hits = self._delta("hit_blocks", int(st.match_hits_blocks))
        if hits:
            c("prefix_cache_match_length_total", float(hits * self.e.cfg.block_size))
        q = self._delta("match_queries", int(st.match_queries))
        if q:
            qb = self._delta("match_query_blocks", int(st.match_query_blocks))
            _rt.metric_histogram_observe("prefix_cache_block_matched_num", float(hits) / q)
            if qb:
                _rt.metric_histogram_observe("prefix_cache_block_matched_rate", float(hits) / qb)
        spec = getattr(self.e, "spec", None)
        if spec is not None:
            for name, attr in (("speculative_num_draft_tokens_total", "n_draft"), ("speculative_num_accepted_tokens_total", "n_accepted"),
                               ("speculative_num_drafts_total", "n_steps")):
                v = getattr(spec, attr, None)
                if v is not None:
                    d = self._delta(name, int(v))
                    if d:
                        c(name, float(d))
        now = time.time()
        if now >= self._next_slow:          # once a second: host-side utilisation
            self._next_slow = now + 1.0
            try:
                import psutil
                g("xllm_cpu_utilization", float(psutil.cpu_percent(interval=None)))
            except Exception:
                pass
            try:
                import torch
                if torch.cuda.is_available():
                    g("xllm_gpu_num", float(torch.cuda.device_count()))
                    free, total = torch.cuda.mem_get_info()
                    g("total_memory_size_in_kilobytes", total / 1024.0)
            except Exception:
                pass
