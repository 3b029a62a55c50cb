"""OpenTelemetry double-write of the metrics logger, the W&B exporter and the rollout traffic routers."""
import pytest

otel = pytest.importorskip("opentelemetry.sdk.metrics")


def test_gauges_and_wandb_exporter():
    from opentelemetry.sdk.metrics import MeterProvider
    from opentelemetry.sdk.metrics.export import InMemoryMetricReader, MetricExportResult
    from tunix_b200.common.configs import MetricsLoggerOptions
    from tunix_b200.sft import metrics_logger as ml
    from tunix_b200.sft.otel_wandb import WandbMetricsExporter, _wandb_payloads
    assert ml.otel_metric_name("loss") == "tunix.training.loss" and ml.otel_metric_name("rewards/mean score") == "tunix.rewards.mean.score"
    assert ml.otel_metric_name("///") == "tunix.unnamed"
    reader = InMemoryMetricReader()
    logger = ml.MetricsLogger(MetricsLoggerOptions(enable_opentelemetry=True), otel_meter_provider=MeterProvider(metric_readers=[reader]))
    logger.log("actor", "loss", 2.5, "train", 7)
    logger.log("actor", "kl", 0.1, "train", 7)
    logger.log("", "loss", 3.0, "eval", 4)
    assert logger.get_metric("actor", "loss", "train") == 2.5                  # the history is unaffected
    data = reader.get_metrics_data()
    payloads = list(_wandb_payloads(data))
    assert payloads == [(4, {"eval/tunix.training.loss": 3.0}), (7, {"actor/train/tunix.training.loss": 2.5, "actor/train/tunix.kl": 0.1})]

    class Run:
        def __init__(self):
            self.calls = []

        def log(self, values, step=None):
            self.calls.append((step, dict(values)))
    run = Run()
    exp = WandbMetricsExporter(run)
    assert exp.export(data) == MetricExportResult.SUCCESS and [s for s, _ in run.calls] == [4, 7]
    assert exp.force_flush() and exp.shutdown() is None

    class Broken:
        def log(self, *a, **k):
            raise IOError("offline")
    assert WandbMetricsExporter(Broken()).export(data) == MetricExportResult.FAILURE
    # without the option nothing is emitted
    reader2 = InMemoryMetricReader()
    ml.MetricsLogger(MetricsLoggerOptions(), otel_meter_provider=MeterProvider(metric_readers=[reader2])).log("a", "loss", 1.0, "train", 0)
    assert reader2.get_metrics_data() is None or not list(_wandb_payloads(reader2.get_metrics_data()))


def test_traffic_routers():
    from tunix_b200.rl.rollout.rollout_traffic_router import (HashTrafficRouter, RolloutTrafficRoutingParams as P,
                                                              RoundRobinTrafficRouter)
    h = HashTrafficRouter(4)
    picks = [h.route(P(trajectory_id=i)) for i in range(64)]
    assert picks == [h.route(P(trajectory_id=i)) for i in range(64)] and set(picks) == {0, 1, 2, 3}
    rr = RoundRobinTrafficRouter(3)
    assert [rr.route(P(trajectory_id=9)) for _ in range(5)] == [0, 1, 2, 0, 1]
    with pytest.raises(ValueError):
        HashTrafficRouter(0)
