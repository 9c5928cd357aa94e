from .base import OmniConnectorBase  # noqa: F401
from .factory import (ConnectorSpec, OmniConnectorFactory, initialize_orchestrator_connectors,  # noqa: F401
                      load_omni_transfer_config)
