from .clients import BtRmClient, GenRmClient, KvStore, KvStoreClient, SamplerClient, TeacherClient  # noqa: F401
from .rpc import HttpRpcClient, LocalRpcClient, RpcClient, pick_endpoint_idx, serve  # noqa: F401
