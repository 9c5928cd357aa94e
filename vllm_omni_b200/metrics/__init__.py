from .stats import (OrchestratorAggregator, RequestE2EStats, StageRequestStats, StageStats,  # noqa: F401
                    TransferEdgeStats)
