# Two 8-GPU nodes: expert parallelism inside each node, data parallelism across them. Both allocations run the same
# line; the node rank is the allocation index and the rendezvous address is the first allocation's host.
job "halo-b200-sft-120b-2node" {
  type = "batch"
  group "trainer" {
    count = 2
    constraint { distinct_hosts = true }
    restart { attempts = 0 }
    network { port "rdzv" { static = 29500 } }
    service { name = "halo-b200-rdzv"  port = "rdzv" }
    task "train" {
      driver = "docker"
      config {
        image        = "halo-b200:latest"
        ipc_mode     = "host"
        network_mode = "host"
        command      = "bash"
        args         = ["-c", "python -m halo_b200.cli launch sft examples/recipes/sft_moe_120b_2node_ep8.yaml -n 8 --numa-binding"]
      }
      template {
        destination = "local/rdzv.env"
        env         = true
        data        = <<EOT
{{ range $i, $s := service "halo-b200-rdzv" }}{{ if eq $i 0 }}HALO_RDZV_ENDPOINT={{ $s.Address }}:{{ $s.Port }}{{ end }}{{ end }}
EOT
      }
      env {
        HALO_NNODES                 = "2"
        HALO_NODE_RANK              = "${NOMAD_ALLOC_INDEX}"
        CUDA_DEVICE_MAX_CONNECTIONS = "1"
        NVLINK_DOMAIN_SIZE          = "8"
      }
      resources {
        cpu    = 64000
        memory = 512000
        device "nvidia/gpu" { count = 8 }
      }
    }
  }
}
