import logging

log = logging.getLogger("hiscache")


class Config(dict):
    """A dict that also answers attribute access, like the OmegaConf objects the reference
    is driven by (example/main.py:13-15 loads them with Hydra from a config tree that is not
    part of the project).  Nested dicts are wrapped on the way in."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        for k, v in dict(*args, **kwargs).items():
            self[k] = v

    def __setitem__(self, k, v):
        if isinstance(v, dict) and not isinstance(v, Config):
            v = Config(v)
        super().__setitem__(k, v)

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v


def cfg_get(cfg, path, default=None):
    """cfg.a.b.c with a default when any level is missing."""
    cur = cfg
    for part in path.split("."):
        try:
            cur = cur[part]
        except (KeyError, TypeError, IndexError):
            return default
    return cur


def make_config(*, feature_dim, num_classes, hidden_dim, num_layers, num_nodes, model="SAGE",
                dropout=0.5, num_device=1, device="cuda:0", feat_mode="history_uvm",
                method="grad", rate=0.5, staleness_thres=10, start_history=0, limit=1.0,
                distributed_store=False, lr=1e-3, num_epochs=1, eval_begin=1 << 30,
                dataset_name="synthetic", dataset_path="", num_rel=1, buffer_size=0,
                batch_size=1000, fanouts=(15, 10, 5), exchange="auto", **extra):
    """Builds the nested config the classes of this package read (the same keys as the
    reference: hiscache/history_cache.py:13-35,58, hiscache/history_table.py:21-30,63,
    hiscache/history_model.py:447-452, hiscache/history_trainer.py:20-40)."""
    cfg = Config(
        dl=dict(dataset=dict(feature_dim=feature_dim, num_classes=num_classes, path=dataset_path,
                             name=dataset_name, num_nodes=num_nodes),
                num_device=num_device, device=device, type="cxg",
                loading=dict(feat_mode=feat_mode), performance=dict(prof=False),
                sampler=dict(batch_size=batch_size, fanouts=list(fanouts))),
        train=dict(type="cxg", model=dict(type=model, hidden_dim=hidden_dim, num_layers=num_layers,
                                          dropout=dropout, num_rel=num_rel),
                   train=dict(num_epochs=num_epochs, eval_begin=eval_begin), optimizer=dict(lr=lr)),
        history=dict(method=method, rate=rate, staleness_thres=staleness_thres,
                     start_history=start_history, limit=limit,
                     distributed_store=distributed_store, buffer_size=buffer_size,
                     store_last_layer=False, graph_struct_norm=0, exchange=exchange),
    )
    for k, v in extra.items():
        cfg[k] = v
    return cfg
