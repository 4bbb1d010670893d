# One 8-GPU node, experts sharded over the eight GPUs.
job "halo-b200-sft-30b-a3b" {
  type = "batch"
  group "trainer" {
    count = 1
    restart { attempts = 0 }
    task "train" {
      driver = "docker"
      config {
        image        = "halo-b200:latest"
        ipc_mode     = "host"
        network_mode = "host"
        command      = "python"
        args         = ["-m", "halo_b200.cli", "launch", "sft", "examples/recipes/sft_moe_30b_a3b_ep8.yaml", "-n", "8", "--numa-binding"]
      }
      env {
        CUDA_DEVICE_MAX_CONNECTIONS = "1"
        HALO_DATA_ROOT              = "/scratch/halo_b200"
      }
      resources {
        cpu    = 64000
        memory = 512000
        device "nvidia/gpu" { count = 8 }
      }
    }
  }
}
