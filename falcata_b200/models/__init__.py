"""Model families: gradient boosting (gbdt), DART, random forest — all driven by the native
``GBDT`` class; sklearn-style estimators live in :mod:`falcata_b200.sklearn`."""
