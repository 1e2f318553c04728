"""Import-compatibility names: ``omni_moe.*`` resolves to the sm_100a implementation in
``omni_moe_b200`` so code written against the reference package's import paths runs unchanged."""
